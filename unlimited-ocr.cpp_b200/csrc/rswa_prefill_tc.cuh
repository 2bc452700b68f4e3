// Ragged prefill attention on the 5th-generation tensor cores (tcgen05 + TMEM), sm_100a.
//
// A work item is a tile of up to 128 consecutive query rows of one request and one head, with the
// 128-key tiles those rows can see: first the fixed (prefix) region through the block table, then --
// for text rows -- the sliding text window in the text pool.  One persistent CTA per SM draws items
// from a global counter, longest first (rswa_prefill_order_kernel orders the tiles by their number of
// key tiles), and keeps its pipeline running across items.  16 warps, warp-specialised, registers
// re-split between the roles with setmaxnreg:
//
//   warps 0-7    softmax: warp w owns rows 32*(w%4).. (its TMEM lane quadrant) and half w/4 of the
//                keys of S: tcgen05.ld of S, scores of hidden keys set to -inf, row maximum agreed with
//                the partner warp through shared memory, exp2-domain probabilities written over S in
//                TMEM (tcgen05.st) as bf16 hi and lo pairs.  The accumulator O stays in TMEM across the
//                item's key tiles; the reference the probabilities are scaled by only follows the row
//                maximum in steps of 2^8, and a row whose reference moved rescales its accumulator row
//                in place before the tile's product is added
//   warps 8-11   helpers, thread r owning row r of a staging area: one bulk copy brings the fp32
//                query row in, the thread splits it into the bf16 hi / lo operand in TMEM (as soon as
//                the previous item's last scores have left the tensor core), later reads the finished
//                accumulator row, normalises it, stages it and sends it off with one bulk store
//   warp 12      K producer and the CTA's scheduler: per key tile 16 tiled TMA loads (one 16-token
//                block half each, SWIZZLE_128B) into a two-deep ring; blocks the rows cannot see are
//                fetched from an out-of-range coordinate, which fills zeros.  Lane 0 draws the items
//                two ahead and publishes them in a shared-memory ring for every other role
//   warp 14      V producer, the same loads for V
//   warp 13      one thread issues S = Q K^T (tcgen05.mma kind::f16, M = N = 128, Q from TMEM, K from
//                shared memory), up to two tiles ahead of the softmax
//   warp 15      one thread issues O += P V (P from TMEM, V as the MN-major shared-memory operand)
//
// Two issuing threads because the tensor core takes one thread's instructions in order and every
// barrier poll between two batches leaves its queue empty for a few hundred cycles: one thread's
// polls are covered by the other's queued instructions.
//
// TMEM (512 columns): S/P double-buffered in [0,256), O in [256,384), Q hi / lo words in [384,512).
//
// The queries arrive in fp32 and the oracle computes in fp32, so Q and P are each fed to the tensor
// cores as a bf16 pair (hi + lo): two MMAs per operand keep ~16 mantissa bits, which holds the
// stated tolerance (rel-L2 1e-3) that a single bf16 rounding of Q would not.  K and V are the cache's
// own bf16 payload.  Semantics: RSWACache::attention (src/scheduler/kv_cache.cpp:84-130) for vision
// rows (causal over the fixed region) and, for text rows, the append-then-attend composition that
// defines "prefix + last W tokens".
//
// Every wait is bounded; a wait that runs out sets a status bit, every role leaves its loop, the
// copies and MMAs in flight are drained (bounded again) and the CTA frees its TMEM.  A parity wait
// only tells a barrier phase from its neighbours: every waiter here follows its barrier phase by
// phase (per key tile, or per item on barriers of its own), never skipping one.
#pragma once

#include <cuda.h>  // CUtensorMap (type only; the encoder is fetched through the runtime)

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

struct TcWork;
struct PrefillParams {
    const float* q;
    float* out;
    int out_bf16;  // 1: `out` holds bf16 rows (round-to-nearest-even), else fp32
    const uint8_t* k_pool;
    const uint8_t* v_pool;
    const uint8_t* k_text;
    const uint8_t* v_text;
    const int32_t* table;
    const int* d_prefill_len;
    const PrefillTile* tiles;
    const struct TcWork* work;  // the tiles with their key-tile counts, most key tiles first (rswa_prefill_order_kernel)
    int* counter;               // items handed out beyond every CTA's first (zero at launch)
    int table_stride, num_blocks, text_blocks;
    int n_tiles;
    int heads, kv_heads, group, window;
    float scale_log2e;
    int* status;
    uint32_t wait_limit;  // polls a wait may take before the role gives up (kWaitLimit unless a test lowers it); the
                          // drains of copies and MMAs in flight keep the full limit
};

constexpr int kTcTile = 128;             // queries per CTA, keys per step, head_dim
constexpr uint32_t kTcColO = 256;        // TMEM columns: S/P buffers at 0 and 128, the accumulator at 256,
constexpr uint32_t kTcColQ = 384;        // Q as bf16 pairs at 384 (hi words) and 448 (lo words)
constexpr int kTcHalfBytes = 128 * 128;  // one 64-element-wide half of a 128x128 bf16 tile
constexpr int kTcTileBytes = 2 * kTcHalfBytes;

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

// Instruction descriptor, kind::f16: D fp32, A and B bf16 (an fp16 A with a bf16 B raised an illegal
// instruction on this part, so both operands keep the cache's type), M = N = 128; B K-major or MN-major.
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

// D[tmem_d] (+)= A * B: A operand from TMEM (lane = row, two bf16 per 32-bit column), B from shared memory.
// acc == 0 overwrites D.
__device__ __forceinline__ void tc_mma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t acc) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.u32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(acc) : "memory");
}

__device__ __forceinline__ void tc_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}

__device__ __forceinline__ void tc_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}

__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// Truncating hi/lo split of two floats into packed bf16 pairs: hi keeps the top 16 bits, lo the top
// 16 bits of the exact remainder, so hi + lo carries 16 mantissa bits of the input.
__device__ __forceinline__ void tc_split2(float a, float b, uint32_t& hi, uint32_t& lo) {
    const uint32_t ua = __float_as_uint(a), ub = __float_as_uint(b);
    hi = __byte_perm(ua, ub, 0x7632);
    const float ra = a - __uint_as_float(ua & 0xffff0000u), rb = b - __uint_as_float(ub & 0xffff0000u);
    lo = __byte_perm(__float_as_uint(ra), __float_as_uint(rb), 0x7632);
}

__device__ __forceinline__ float tc_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}


__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// Tiled TMA load of one box (64 elements x 16 rows of a [rows][128] bf16 matrix) into shared memory.
// x (innermost coordinate) is 0 or 64: a multiple of 16 bytes as the engine requires.  A row
// coordinate at or beyond the matrix's extent fills the box with zeros and still completes the full
// byte count on the barrier.
__device__ __forceinline__ void tma_load_box(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::
            "r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar)
        : "memory");
}

// shared -> global bulk copy of this thread's bulk-async group.  Both addresses and the size are multiples of 16 bytes.
__device__ __forceinline__ void bulk_copy_s2g(void* dst, uint32_t src, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(__cvta_generic_to_global(dst)), "r"(src), "r"(bytes)
                 : "memory");
}

struct PrefillMaps {
    CUtensorMap k, v;    // paged pool, as a [num_blocks * kv_heads * 16][128] bf16 matrix
    CUtensorMap tk, tv;  // text pool, same shape with text_blocks
};


constexpr int kTcSoftmaxThreads = 256;  // warps 0-7: warp w owns rows 32*(w%4).., key/dim half w/4
constexpr int kTcHelperThreads = 128;   // warps 8-11: thread r moves row r (Q in, output out)
constexpr int kTcThreads = 512;         // + warp 12 K producer, 13 S issuer and TMEM owner, 14 V producer, 15 O issuer
constexpr int kTcExchangeBytes = (2 * 2 * 128 + 2 * 2 * 128) * 4;  // row-max exchange (by tile parity) + row sums (by item parity)
constexpr int kTcStages = 2;                                   // depth of the K and of the V ring
constexpr uint32_t kTcStageBytes = 2 * kTcTileBytes;           // one K tile + one V tile
constexpr uint32_t kTcQRowBytes = 528;                         // a staged fp32 row: 512 bytes + 16, so that row-owning and row-wide accesses are conflict-free
constexpr uint32_t kTcQStageBytes = 128 * kTcQRowBytes;
constexpr int kTcSmemBytes = kTcStages * kTcStageBytes + kTcQStageBytes + 512 + 512 + kTcExchangeBytes + 1024;  // K/V ring, Q / output staging, barriers, item ring, exchange, alignment slack

// 64 consecutive TMEM columns of this thread's lane into registers: two loads, one wait.  The wait
// and the empty statement after it name the registers so that no use can be scheduled before them.
#define UOCR_R32(r, o) "=r"(r[o + 0]), "=r"(r[o + 1]), "=r"(r[o + 2]), "=r"(r[o + 3]), "=r"(r[o + 4]), "=r"(r[o + 5]), "=r"(r[o + 6]), "=r"(r[o + 7]), \
    "=r"(r[o + 8]), "=r"(r[o + 9]), "=r"(r[o + 10]), "=r"(r[o + 11]), "=r"(r[o + 12]), "=r"(r[o + 13]), "=r"(r[o + 14]), "=r"(r[o + 15]), \
    "=r"(r[o + 16]), "=r"(r[o + 17]), "=r"(r[o + 18]), "=r"(r[o + 19]), "=r"(r[o + 20]), "=r"(r[o + 21]), "=r"(r[o + 22]), "=r"(r[o + 23]), \
    "=r"(r[o + 24]), "=r"(r[o + 25]), "=r"(r[o + 26]), "=r"(r[o + 27]), "=r"(r[o + 28]), "=r"(r[o + 29]), "=r"(r[o + 30]), "=r"(r[o + 31])
#define UOCR_RW32(r, o) "+r"(r[o + 0]), "+r"(r[o + 1]), "+r"(r[o + 2]), "+r"(r[o + 3]), "+r"(r[o + 4]), "+r"(r[o + 5]), "+r"(r[o + 6]), "+r"(r[o + 7]), \
    "+r"(r[o + 8]), "+r"(r[o + 9]), "+r"(r[o + 10]), "+r"(r[o + 11]), "+r"(r[o + 12]), "+r"(r[o + 13]), "+r"(r[o + 14]), "+r"(r[o + 15]), \
    "+r"(r[o + 16]), "+r"(r[o + 17]), "+r"(r[o + 18]), "+r"(r[o + 19]), "+r"(r[o + 20]), "+r"(r[o + 21]), "+r"(r[o + 22]), "+r"(r[o + 23]), \
    "+r"(r[o + 24]), "+r"(r[o + 25]), "+r"(r[o + 26]), "+r"(r[o + 27]), "+r"(r[o + 28]), "+r"(r[o + 29]), "+r"(r[o + 30]), "+r"(r[o + 31])
#define UOCR_LD32_ASM                                                                                          \
    "tcgen05.ld.sync.aligned.32x32b.x32.b32 "                                                                  \
    "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "                                   \
    "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"

__device__ __forceinline__ void tc_ld64(uint32_t taddr, uint32_t (&r)[64]) {
    asm volatile(UOCR_LD32_ASM : UOCR_R32(r, 0) : "r"(taddr));
    asm volatile(UOCR_LD32_ASM : UOCR_R32(r, 32) : "r"(taddr + 32));
    asm volatile("tcgen05.wait::ld.sync.aligned;" : UOCR_RW32(r, 0) : : "memory");
    asm volatile("" : UOCR_RW32(r, 32) : : "memory");
}

// Bounded rendezvous of the 64 threads that share a TMEM lane quadrant (one mbarrier phase per call).
__device__ __forceinline__ bool pair_sync(uint32_t bar, uint32_t parity, int* status, uint32_t limit) {
    mbar_arrive(bar);
    return __all_sync(0xffffffffu, mbar_wait_bounded(bar, parity, status, limit));
}

// How far a row's maximum may rise above the reference its probabilities are scaled by before the
// reference moves (in the exp2 domain: probabilities stay below 2^8).  The O accumulator lives in TMEM
// across key tiles; moving a row's reference means rescaling that row of it, so the reference only
// follows the maximum in steps.
constexpr float kTcMaxSlack = 8.f;

// One key tile of the online softmax for this thread: its row, its half (64 keys) of the tile.
// Reads S once, agrees on the row maximum with the thread that owns the other half (shared-memory
// exchange + a 64-thread rendezvous), writes P as bf16 pairs over its own 64 columns of the S buffer:
// 32 words of hi pairs, then 32 words of lo pairs.  full (the same for the whole warp): every key of the
// tile is visible to every row of the warp; otherwise the scores of the keys outside [vlo, vhi) are
// set to -inf first (their probabilities come out as zero), so that both cases run the same code.
// m_ref is the reference the row's probabilities are scaled by; alpha is the factor the row's
// accumulator and sum take when the reference moved (1 otherwise).  False if the rendezvous ran out
// of time.
__device__ __forceinline__ bool tc_softmax_half(bool full, uint32_t tS, int h, int vlo, int vhi, float* my_max, const float* other_max,
                                                uint32_t pair_bar, uint32_t pair_parity, int* status, uint32_t wait_limit,
                                                float& m_ref, float& l_run, float& alpha) {
    uint32_t s[64];
    tc_ld64(tS + h * 64, s);
    if (!full) {
        // Of this thread's 64 keys the visible ones are [lo, hi).  A causal edge only has an upper bound, a window
        // edge only a lower one: each bound is applied only where some row of the warp needs it.
        const int lo = vlo - h * 64, hi = vhi - h * 64;
        if (__any_sync(0xffffffffu, hi < 64)) {
#pragma unroll
            for (int j = 0; j < 64; ++j)
                if (j >= hi) s[j] = 0xff800000u;  // -inf
        }
        if (__any_sync(0xffffffffu, lo > 0)) {
#pragma unroll
            for (int j = 0; j < 64; ++j)
                if (j < lo) s[j] = 0xff800000u;
        }
    }
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < 64; ++j) mx = fmaxf(mx, __uint_as_float(s[j]));
    *my_max = mx;
    // also: both halves of S are in registers from here on, P may overwrite them
    if (!pair_sync(pair_bar, pair_parity, status, wait_limit)) return false;
    // both threads of the row see the same two maxima and take the same decision
    const float m_tile = fmaxf(mx, *other_max);
    alpha = 1.f;
    if (m_tile > m_ref + kTcMaxSlack) {  // also the first visible key of the row (m_ref = -inf)
        alpha = tc_exp2(m_ref - m_tile);
        m_ref = m_tile;
    }
    const float m_safe = (m_ref == -INFINITY) ? 0.f : m_ref;
    float lsum = 0.f;
#pragma unroll
    for (int qq = 0; qq < 2; ++qq) {  // 32 keys at a time: their 16 hi words, then their 16 lo words, over their own columns
        uint32_t pk[32];
#pragma unroll
        for (int e = 0; e < 16; ++e) {
            const float p0 = tc_exp2(__uint_as_float(s[qq * 32 + 2 * e]) - m_safe);
            const float p1 = tc_exp2(__uint_as_float(s[qq * 32 + 2 * e + 1]) - m_safe);
            lsum += p0 + p1;
            tc_split2(p0, p1, pk[e], pk[16 + e]);
        }
        tc_st32(tS + h * 64 + qq * 32, pk);
    }
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
    l_run = l_run * alpha + lsum;
    return true;
}

// This thread's 64 dims of its accumulator row in TMEM times alpha, in place.
__device__ __forceinline__ void tc_rescale(uint32_t tO, float alpha) {
    uint32_t o[64];
    tc_ld64(tO, o);
    uint32_t w[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) w[j] = __float_as_uint(__uint_as_float(o[j]) * alpha);
    tc_st32(tO, w);
#pragma unroll
    for (int j = 0; j < 32; ++j) w[j] = __float_as_uint(__uint_as_float(o[32 + j]) * alpha);
    tc_st32(tO + 32, w);
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// A query tile with the key tiles its rows can see, as the ordering kernel leaves it for the persistent grid.
struct TcWork {
    PrefillTile t;
    int pfx;             // the slot's fixed-region length
    int n_prefix_tiles;  // key tiles in the fixed region, then (text rows) in the text window from tile text_tile0
    int text_tile0;
    int n_steps;
    int pad[2];
};
static_assert(sizeof(TcWork) == 48, "three 16-byte loads");

// One work item of the persistent grid: a query tile and a head.
struct TcItem {
    PrefillTile t;
    int head, kvh;
    int pfx, n_prefix_tiles, text_tile0, n_steps;
    bool valid;
};
constexpr int kTcItemSlots = 8;  // items the CTA's scheduler may have published and not every role has read
constexpr int kTcItemInts = 16;  // ints per published item

// Key tiles the rows of query tile t can see: the fixed region (causal for vision rows), then, for text rows,
// the text window.
__device__ __forceinline__ void tc_tile_steps(const PrefillTile& t, int pfx, int window, int& n_prefix_tiles, int& text_tile0, int& n_steps) {
    const int plim = t.kind == 0 ? min(t.pos0 + t.rows, pfx) : pfx;
    n_prefix_tiles = (plim + kTcTile - 1) / kTcTile;
    text_tile0 = 0;
    int n_text_tiles = 0;
    if (t.kind == 1) {
        text_tile0 = max(0, t.pos0 - window + 1) / kTcTile;
        n_text_tiles = (t.pos0 + t.rows - 1) / kTcTile - text_tile0 + 1;
    }
    n_steps = n_prefix_tiles + n_text_tiles;
}

// Orders the query tiles by their number of key tiles, most first (a counting sort in one CTA; the order within
// one count is arbitrary), and leaves each with its counts in `work`.  The persistent grid hands out (tile, head)
// items in this order, heads innermost: CTA c starts with item c, the counter (zero at launch) gives the rest.
constexpr int kTcOrderBins = 256;
__global__ void __launch_bounds__(256) rswa_prefill_order_kernel(const PrefillParams p, TcWork* work) {
    __shared__ int hist[kTcOrderBins];
    auto work_of = [&](int i) {
        TcWork w;
        w.t = p.tiles[i];
        w.pfx = max(__ldg(p.d_prefill_len + w.t.slot), 0);
        tc_tile_steps(w.t, w.pfx, p.window, w.n_prefix_tiles, w.text_tile0, w.n_steps);
        w.pad[0] = w.pad[1] = 0;
        return w;
    };
    for (int i = threadIdx.x; i < kTcOrderBins; i += blockDim.x) hist[i] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < p.n_tiles; i += blockDim.x) atomicAdd(&hist[min(work_of(i).n_steps, kTcOrderBins - 1)], 1);
    __syncthreads();
    if (threadIdx.x == 0) {  // first index of each count, largest count first
        int at = 0;
        for (int b = kTcOrderBins - 1; b >= 0; --b) {
            const int n = hist[b];
            hist[b] = at;
            at += n;
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < p.n_tiles; i += blockDim.x) {
        const TcWork w = work_of(i);
        work[atomicAdd(&hist[min(w.n_steps, kTcOrderBins - 1)], 1)] = w;
    }
}

// Register budget of the roles (setmaxnreg): the kernel starts with 65536 / 512 = 128 registers per thread; the
// issuing / producing warps and the helper warps hand most of theirs back, the softmax warps take them.
#define UOCR_TC_REGS_SOFTMAX 168
#define UOCR_TC_REGS_HELPER 104
#define UOCR_TC_REGS_ISSUE 64

__global__ void __launch_bounds__(kTcThreads, 1)
rswa_prefill_tc_kernel(const PrefillParams p, const __grid_constant__ PrefillMaps maps) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sKV = base;                               // stage b: K at sKV + b * kTcStageBytes, V one tile after it
    uint8_t* sQ = base + kTcStages * kTcStageBytes;    // fp32 query rows on their way to TMEM, then the output rows
    uint64_t* bars = reinterpret_cast<uint64_t*>(sQ + kTcQStageBytes);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 30);
    int* item_ring = reinterpret_cast<int*>(bars + 64);                              // [kTcItemSlots][kTcItemInts]
    float* xmax = reinterpret_cast<float*>(item_ring + kTcItemSlots * kTcItemInts);  // [tile parity][half][row]
    float* xsum = xmax + 2 * 2 * 128;                                                // [item parity][half][row]
    const uint32_t bar0 = smem_addr(bars);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // Ring and S/P barriers are indexed by the parity of the CTA's running key-tile count g; their phase is (g >> 1) & 1.
    auto k_full = [&](uint32_t b) { return bar0 + (0 + b) * 8; };   // TMA bytes of K stage b have landed
    auto k_free = [&](uint32_t b) { return bar0 + (2 + b) * 8; };   // the S MMAs reading K stage b are done
    auto v_full = [&](uint32_t b) { return bar0 + (4 + b) * 8; };   // same for V and the O MMAs
    auto v_free = [&](uint32_t b) { return bar0 + (6 + b) * 8; };
    auto s_full = [&](uint32_t b) { return bar0 + (8 + b) * 8; };   // S buffer b holds Q K^T
    auto p_full = [&](uint32_t b) { return bar0 + (10 + b) * 8; };  // all 256 softmax threads wrote their P over S buffer b
    auto o_full = [&](uint32_t b) { return bar0 + (12 + b) * 8; };  // the accumulator holds the products up to a tile of parity b
    // Per item m.  A waiter can be one item behind the arrivals of q_full and l_ready, never two, so these are
    // indexed by m & 1 with phase (m >> 1) & 1; the others are one barrier with phase m & 1.
    const uint32_t q_landed = bar0 + 14 * 8;                          // the item's query rows are in the staging area
    auto q_full = [&](uint32_t m) { return bar0 + (16 + (m & 1u)) * 8; };   // Q of item m is in TMEM
    auto l_ready = [&](uint32_t m) { return bar0 + (18 + (m & 1u)) * 8; };  // the row sums of item m are in xsum
    const uint32_t o_read = bar0 + 15 * 8;                            // the helpers hold item m's accumulator rows in registers
    // A parity wait only tells a phase from its neighbours, so the helpers (who do not follow the key tiles) get
    // the end of an item's S products and of its P V products as barriers of their own, one phase per item.
    const uint32_t s_done = bar0 + 26 * 8, o_done = bar0 + 27 * 8;
    const uint32_t drained = bar0 + 24 * 8, drained2 = bar0 + 25 * 8; // the issuers' last instructions have completed
    auto pair_bar = [&](int quad) { return bar0 + (20 + quad) * 8; };  // the two softmax warps of a lane quadrant
    // The CTA's items come from a global counter: the K producer draws them two items ahead of its own loads and
    // publishes each in a ring slot; every other role reads the slot when it gets to the item.  item_full: slot
    // written; item_empty: every reading warp (8 softmax, 4 helper, V producer, the two issuers) has read it.
    auto item_full = [&](uint32_t sl) { return bar0 + (32 + sl) * 8; };
    auto item_empty = [&](uint32_t sl) { return bar0 + (40 + sl) * 8; };
    constexpr uint32_t kItemReaders = 8 + 4 + 1 + 1 + 1;
    auto read_slot = [&](uint32_t sl) {
        const int* w = item_ring + sl * kTcItemInts;
        TcItem it;
        it.t.row0 = w[0]; it.t.rows = w[1]; it.t.slot = w[2]; it.t.kind = w[3]; it.t.pos0 = w[4]; it.t.block0 = w[5];
        it.head = w[6]; it.pfx = w[7]; it.n_prefix_tiles = w[8]; it.text_tile0 = w[9]; it.n_steps = w[10];
        it.valid = w[11] != 0;
        it.kvh = it.head / p.group;
        if (!it.valid) it.n_steps = 0;
        return it;
    };
    auto no_item = [&]() {
        TcItem it;
        it.valid = false;
        it.n_steps = 0;
        it.t.rows = 0;
        return it;
    };
    // the j-th item of this CTA, for a whole warp / for a single thread; invalid after the last one (or a wait that ran out)
    auto get_item = [&](uint32_t j) {
        const uint32_t sl = j % kTcItemSlots;
        if (!__all_sync(0xffffffffu, mbar_wait_bounded(item_full(sl), (j / kTcItemSlots) & 1u, p.status, p.wait_limit))) return no_item();
        const TcItem it = read_slot(sl);
        __syncwarp();
        if (lane == 0) mbar_arrive(item_empty(sl));
        return it;
    };
    auto get_item_1 = [&](uint32_t j) {
        const uint32_t sl = j % kTcItemSlots;
        if (!mbar_wait_bounded(item_full(sl), (j / kTcItemSlots) & 1u, p.status, p.wait_limit)) return no_item();
        const TcItem it = read_slot(sl);
        mbar_arrive(item_empty(sl));
        return it;
    };

    if (tid == 0) {
#pragma unroll
        for (int b = 0; b < 2; ++b) {
            mbar_init(k_full(b), 1);
            mbar_init(k_free(b), 1);
            mbar_init(v_full(b), 1);
            mbar_init(v_free(b), 1);
            mbar_init(s_full(b), 1);
            mbar_init(p_full(b), kTcSoftmaxThreads);
            mbar_init(o_full(b), 1);
            mbar_init(q_full(b), kTcHelperThreads);
            mbar_init(l_ready(b), kTcSoftmaxThreads);
        }
        mbar_init(q_landed, kTcHelperThreads);
        mbar_init(o_read, kTcHelperThreads);
        mbar_init(s_done, 1);
        mbar_init(o_done, 1);
        mbar_init(drained, 1);
        mbar_init(drained2, 1);
#pragma unroll
        for (int sl = 0; sl < kTcItemSlots; ++sl) {
            mbar_init(item_full(sl), 1);
            mbar_init(item_empty(sl), kItemReaders);
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) mbar_init(pair_bar(q), 64);
        mbar_init_fence();
    }
    if (warp == 13) {  // 512 TMEM columns: S/P buffers at 0 and 128, the accumulator at 256, Q at 384
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(tmem_slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot;

    // Register hand-over: every warp of a warpgroup (warps 0-3, 4-7, 8-11, 12-15) executes the same instruction.
    if (warp < 8) {
        // ================= softmax warps ==============================================================
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(UOCR_TC_REGS_SOFTMAX));
        const int quad = warp & 3, h = warp >> 2;  // TMEM lane quadrant; key half of S and dim half of O
        const int r = quad * 32 + lane;            // query row of the tile == TMEM lane
        const uint32_t lane_base = (uint32_t)(quad * 32) << 16;
        const uint32_t tO = tmem + lane_base + kTcColO + h * 64;  // this thread's 64 dims of its accumulator row
        uint32_t g = 0;    // key tiles this CTA has gone through
        uint32_t itc = 0;  // items this CTA has gone through
        uint32_t pp = 0;   // rendezvous of the warp pair so far
        bool ok = true;
        for (TcItem cur = get_item(0); cur.valid && ok; cur = get_item(++itc)) {
            const PrefillTile& t = cur.t;
            const bool live = r < t.rows;
            const int i = t.pos0 + r;
            const int phi = !live ? 0 : (t.kind == 0 ? min(i + 1, cur.pfx) : cur.pfx);  // fixed-region tokens [0, phi)
            const int tlo = max(0, i - p.window + 1);
            const int thi = (live && t.kind == 1) ? i + 1 : 0;                           // text tokens [tlo, thi)
            // Q of this item is in TMEM: the helpers have also taken the sums of the item before last out of xsum
            if (!__all_sync(0xffffffffu, mbar_wait_bounded(q_full(itc), (itc >> 1) & 1u, p.status, p.wait_limit))) { ok = false; break; }
            float m_ref = -INFINITY, l_run = 0.f;
            for (int n = 0; n < cur.n_steps; ++n) {
                const uint32_t gn = g + n, b = gn & 1u, par = (gn >> 1) & 1u;
                const bool text = n >= cur.n_prefix_tiles;
                const int t0 = text ? (cur.text_tile0 + n - cur.n_prefix_tiles) * kTcTile : n * kTcTile;
                const int vlo = text ? tlo - t0 : -(1 << 30);
                const int vhi = (text ? thi : phi) - t0;
                // warp-uniform outcome: the TMEM instructions below need the whole warp
                if (!__all_sync(0xffffffffu, mbar_wait_bounded(s_full(b), par, p.status, p.wait_limit))) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t tS = tmem + lane_base + b * 128;
                float* my_max = xmax + (b * 2 + h) * 128 + r;
                const float* other_max = xmax + (b * 2 + (h ^ 1)) * 128 + r;
                float alpha = 1.f;
                const bool full = __all_sync(0xffffffffu, vlo <= 0 && vhi >= kTcTile);
                ok = tc_softmax_half(full, tS, h, vlo, vhi, my_max, other_max, pair_bar(quad), pp & 1u, p.status, p.wait_limit, m_ref, l_run, alpha);
                ++pp;
                if (!ok) break;
                // A row whose reference moved takes the factor on its accumulator before this tile's product is
                // added: the previous product must have landed, and this tile's P is only announced afterwards.
                if (n >= 1 && __any_sync(0xffffffffu, alpha != 1.f)) {
                    const uint32_t gk = gn - 1;
                    if (!__all_sync(0xffffffffu, mbar_wait_bounded(o_full(gk & 1u), (gk >> 1) & 1u, p.status, p.wait_limit))) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    tc_rescale(tO, alpha);
                }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                mbar_arrive(p_full(b));
            }
            if (!ok) break;
            // the row's sum over this thread's key half goes to the helper that writes the row out
            xsum[((itc & 1u) * 2 + h) * 128 + r] = l_run;
            mbar_arrive(l_ready(itc));
            g += cur.n_steps;
        }
    } else if (warp < 12) {
        // ================= helper warps: Q into TMEM, accumulator rows out ==============================
        // Thread r owns row r of the staging area for the whole kernel: it fetches the query row into it (one
        // bulk copy), splits the row into the bf16 hi / lo operand in TMEM, later stages the finished output
        // row there and sends it off with one bulk store -- so the staging area needs no barrier of its own.
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(UOCR_TC_REGS_HELPER));
        const int quad = warp & 3;
        const int r = quad * 32 + lane;
        const uint32_t lane_base = (uint32_t)(quad * 32) << 16;
        uint8_t* my_row = sQ + (size_t)r * kTcQRowBytes;
        const uint32_t my_row_s = smem_addr(my_row);
        uint32_t fetched = 0;  // query-row fetches so far (phases of q_landed begun)
        auto fetch_q = [&](const TcItem& it) {  // this thread's share of the arrivals on q_landed, with its row's bytes
            if (!it.valid) return;
            ++fetched;
            if (r < it.t.rows) {
                mbar_arrive_expect_tx(q_landed, 512u);
                bulk_copy_g2s(my_row_s, p.q + ((size_t)(it.t.row0 + r) * p.heads + it.head) * kTcTile, 512u, q_landed);
            } else {
                mbar_arrive(q_landed);
            }
        };
        // Q row of item m -> TMEM (lane = row, column c of a 64-column block = dims 2c, 2c+1; hi words, then lo words)
        auto convert_q = [&](const TcItem& it, uint32_t m) -> bool {
            if (!__all_sync(0xffffffffu, mbar_wait_bounded(q_landed, m & 1u, p.status, p.wait_limit))) return false;
            const bool live = r < it.t.rows;
            const float s = p.scale_log2e;
            const float4* q4 = reinterpret_cast<const float4*>(my_row);
#pragma unroll 1
            for (int g4 = 0; g4 < 4; ++g4) {  // 32 dims at a time: 16 hi words and 16 lo words (rolled: this runs once per item)
                uint32_t hi[16], lo[16];
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    const float4 v = live ? q4[g4 * 8 + c] : make_float4(0.f, 0.f, 0.f, 0.f);
                    tc_split2(v.x * s, v.y * s, hi[2 * c], lo[2 * c]);
                    tc_split2(v.z * s, v.w * s, hi[2 * c + 1], lo[2 * c + 1]);
                }
                tc_st16(tmem + lane_base + kTcColQ + g4 * 16, hi);
                tc_st16(tmem + lane_base + kTcColQ + 64 + g4 * 16, lo);
            }
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            mbar_arrive(q_full(m));
            return true;
        };

        // Round m: the next item's Q into TMEM, item m's rows out, the query row of the item after next fetched.
        // The first round (m = -1) has no current item: it only brings in Q of item 0 and fetches item 1's rows.
        int m = -1;
        TcItem cur = no_item();
        TcItem nxt = get_item(0);
        bool ok = true;
        fetch_q(nxt);
        while (ok) {
            const TcItem nxt2 = nxt.valid ? get_item((uint32_t)(m + 2)) : no_item();
            // ---- the next item's Q, as soon as this item's last scores have left the tensor core ----------
            if (cur.valid && !__all_sync(0xffffffffu, mbar_wait_bounded(s_done, (uint32_t)m & 1u, p.status, p.wait_limit))) { ok = false; break; }
            if (nxt.valid) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                ok = convert_q(nxt, (uint32_t)(m + 1));
                if (!ok) break;
            }
            if (cur.valid) {
            // ---- this item's row: accumulator / row sum -> staging area -> global -------------------------
            const uint32_t um = (uint32_t)m;
            if (!__all_sync(0xffffffffu, mbar_wait_bounded(l_ready(um), (um >> 1) & 1u, p.status, p.wait_limit))) { ok = false; break; }
            const float l_tot = xsum[((um & 1u) * 2 + 0) * 128 + r] + xsum[((um & 1u) * 2 + 1) * 128 + r];
            const float inv = l_tot > 0.f ? 1.f / l_tot : 0.f;
            if (!__all_sync(0xffffffffu, mbar_wait_bounded(o_done, um & 1u, p.status, p.wait_limit))) { ok = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
            for (int hh = 0; hh < 2; ++hh) {  // (rolled: once per item)
                uint32_t o[64];
                if (cur.n_steps > 0) {
                    tc_ld64(tmem + lane_base + kTcColO + hh * 64, o);
                } else {
#pragma unroll
                    for (int d = 0; d < 64; ++d) o[d] = 0u;
                }
                if (hh == 1) {  // both halves are in registers: the next item's first product may overwrite the accumulator
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    mbar_arrive(o_read);
                }
                if (p.out_bf16) {
                    uint4* so = reinterpret_cast<uint4*>(my_row) + hh * 8;
#pragma unroll
                    for (int c = 0; c < 8; ++c)
                        so[c] = make_uint4(pack_bf16x2(__uint_as_float(o[8 * c]) * inv, __uint_as_float(o[8 * c + 1]) * inv),
                                           pack_bf16x2(__uint_as_float(o[8 * c + 2]) * inv, __uint_as_float(o[8 * c + 3]) * inv),
                                           pack_bf16x2(__uint_as_float(o[8 * c + 4]) * inv, __uint_as_float(o[8 * c + 5]) * inv),
                                           pack_bf16x2(__uint_as_float(o[8 * c + 6]) * inv, __uint_as_float(o[8 * c + 7]) * inv));
                } else {
                    float4* so = reinterpret_cast<float4*>(my_row) + hh * 16;
#pragma unroll
                    for (int c = 0; c < 16; ++c)
                        so[c] = make_float4(__uint_as_float(o[4 * c]) * inv, __uint_as_float(o[4 * c + 1]) * inv,
                                            __uint_as_float(o[4 * c + 2]) * inv, __uint_as_float(o[4 * c + 3]) * inv);
                }
            }
            // this thread's generic-proxy stores -> the bulk store's reads
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            if (r < cur.t.rows) {
                const size_t at = ((size_t)(cur.t.row0 + r) * p.heads + cur.head) * kTcTile;
                if (p.out_bf16)
                    bulk_copy_s2g(reinterpret_cast<uint16_t*>(p.out) + at, my_row_s, 256u);
                else
                    bulk_copy_s2g(p.out + at, my_row_s, 512u);
            }
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            // the row has been read out of the staging area: it takes the query row of the item after next
            asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
            } else {
                // (first round) this thread's reads of its row in convert_q -> the bulk copy that overwrites it
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            }
            fetch_q(nxt2);
            if (!nxt.valid) break;
            ++m;
            cur = nxt;
            nxt = nxt2;
        }
        // after a wait that ran out a fetched query row may still be on its way into the staging area: see it land
        if (!ok && fetched > 0) mbar_wait_bounded(q_landed, (fetched - 1) & 1u, nullptr);
        // the output rows are written before the kernel ends
        asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    } else {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(UOCR_TC_REGS_ISSUE));
    if (warp == 12 || warp == 14) {
        // ================= producer warps: warp 12 feeds K, warp 14 feeds V ===========================
        // lane = (64-dim half, block of the tile).  The ring runs on across items, so the first tiles of the
        // next item are fetched while the current one finishes.
        const int is_v = warp == 14 ? 1 : 0;
        const int blk_i = lane & 7, half = (lane >> 3) & 1;
        const int pool_rows = p.num_blocks * p.kv_heads * kBlockTokens;
        const int text_rows = p.text_blocks * p.kv_heads * kBlockTokens;
        uint32_t g = 0, m = 0, issued = 0;
        bool ok = true;
        // The K producer is also the CTA's scheduler (lane 0): item j of this CTA is the global item k_next -- the
        // CTA's own index for its first, then whatever the counter gives -- written with its tile's data into ring
        // slot j % kTcItemSlots.  The draw for the following item is started right away, its answer is only looked
        // at when that item is published.
        uint32_t pub = 0;
        long long k_next = blockIdx.x;
        bool more = true;
        const long long n_items = (long long)p.n_tiles * p.heads;
        auto publish_one = [&]() -> bool {  // lane 0 only
            const uint32_t sl = pub % kTcItemSlots;
            if (pub >= kTcItemSlots && !mbar_wait_bounded(item_empty(sl), ((pub / kTcItemSlots) - 1) & 1u, p.status, p.wait_limit)) return false;
            int* w = item_ring + sl * kTcItemInts;
            const bool valid = k_next < n_items;
            if (valid) {
                const int ti = (int)(k_next / p.heads);
                const int4* src = reinterpret_cast<const int4*>(p.work + ti);
                const int4 a = __ldg(src), b4 = __ldg(src + 1), c = __ldg(src + 2);
                reinterpret_cast<int4*>(w)[0] = a;                                        // row0 rows slot kind
                reinterpret_cast<int4*>(w)[1] = make_int4(b4.x, b4.y, (int)(k_next - (long long)ti * p.heads), b4.z);  // pos0 block0 head pfx
                reinterpret_cast<int4*>(w)[2] = make_int4(b4.w, c.x, c.y, 1);             // n_prefix_tiles text_tile0 n_steps valid
            } else {
                w[11] = 0;
                more = false;
            }
            mbar_arrive(item_full(sl));  // (release: the slot's contents are visible to whoever sees the phase)
            ++pub;
            if (valid) k_next = (long long)gridDim.x + atomicAdd(p.counter, 1);
            return true;
        };
        for (;; ++m) {
            TcItem it;
            if (is_v) {
                it = get_item(m);
            } else {
                // publish up to item m + 2, then read item m from its slot
                if (lane == 0)
                    while (ok && more && pub < m + 3) ok = publish_one();
                ok = __all_sync(0xffffffffu, ok);
                it = ok ? read_slot(m % kTcItemSlots) : no_item();
            }
            if (!it.valid || !ok) break;
            const int prefix_blocks = (it.pfx + kBlockTokens - 1) / kBlockTokens;
            for (int n = 0; n < it.n_steps; ++n) {
                const uint32_t gn = g + n, b = gn & 1u;
                const uint32_t full = is_v ? v_full(b) : k_full(b), freed = is_v ? v_free(b) : k_free(b);
                if (gn >= 2 && !__all_sync(0xffffffffu, mbar_wait_bounded(freed, ((gn >> 1) - 1) & 1u, p.status, p.wait_limit))) { ok = false; break; }
                const bool text = n >= it.n_prefix_tiles;
                const int t0 = text ? (it.text_tile0 + n - it.n_prefix_tiles) * kTcTile : n * kTcTile;
                const int idx = t0 / kBlockTokens + blk_i;  // block index within the request's region
                int y;
                const CUtensorMap* map;
                if (text) {
                    const int blk = it.t.block0 + idx;
                    y = blk < p.text_blocks ? (blk * p.kv_heads + it.kvh) * kBlockTokens : text_rows;
                    map = is_v ? &maps.tv : &maps.tk;
                } else {
                    y = pool_rows;
                    if (idx < prefix_blocks && idx < p.table_stride) {
                        const int blk = __ldg(p.table + (size_t)it.t.slot * p.table_stride + idx);
                        if (blk < 0 || blk >= p.num_blocks)
                            atomicOr(p.status, kStatusBadBlock);
                        else
                            y = (blk * p.kv_heads + it.kvh) * kBlockTokens;
                    }
                    map = is_v ? &maps.v : &maps.k;
                }
                if (lane == 0) mbar_arrive_expect_tx(full, kTcTileBytes);
                __syncwarp();
                const uint32_t dst = smem_addr(sKV) + b * kTcStageBytes + is_v * kTcTileBytes + half * kTcHalfBytes + blk_i * 2048;
                if (lane < 16) tma_load_box(dst, map, half * 64, y, full);
                issued = gn + 1;
            }
            g += it.n_steps;
        }
        // the last two stages may still be landing if a consumer gave up: wait for them before leaving
        for (uint32_t gn = issued >= 2 ? issued - 2 : 0; gn < issued; ++gn)
            mbar_wait_bounded(is_v ? v_full(gn & 1u) : k_full(gn & 1u), (gn >> 1) & 1u, p.status);
    } else if (warp == 13) {
        // ================= S issuer: one thread issues the Q K^T products ==============================
        // The tensor core takes the instructions of one thread in order, and every barrier poll between two
        // batches leaves its queue empty for a few hundred cycles; with the S and the P V products coming
        // from two threads, one's polls are covered by the other's queued instructions.
        if (lane == 0) {
            const uint32_t idesc_s = tc_instr_desc(false);
            // Every operand descriptor is fixed for the CTA's lifetime except for the ring stage, which only
            // moves the address field: build them once, so that one MMA costs the issuing thread one
            // instruction and an add (the issue loops stay unrolled: rolled, with the descriptor arithmetic in
            // the loop, the thread could not keep the tensor core's queue filled).
            uint64_t dK[8];
#pragma unroll
            for (int j = 0; j < 8; ++j)
                dK[j] = tc_smem_desc(smem_addr(sKV) + (uint32_t)((j >> 2) * kTcHalfBytes + (j & 3) * 32), 16, 1024);
            uint32_t g = 0, m = 0;
            bool ok = true;
            for (TcItem it = get_item_1(0); it.valid && ok; it = get_item_1(++m)) {
                if (!mbar_wait_bounded(q_full(m), (m >> 1) & 1u, p.status, p.wait_limit)) { ok = false; break; }
                for (int n = 0; n < it.n_steps; ++n) {
                    const uint32_t gn = g + n, b = gn & 1u;
                    if (!mbar_wait_bounded(k_full(b), (gn >> 1) & 1u, p.status, p.wait_limit)) { ok = false; break; }
                    // S buffer b held P of the tile two back: the product that read it must have completed
                    if (gn >= 2 && !mbar_wait_bounded(o_full(b), ((gn >> 1) - 1) & 1u, p.status, p.wait_limit)) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint64_t stage = (uint64_t)(b * (kTcStageBytes >> 4));  // address field counts 16-byte units
                    const uint32_t tS = tmem + b * 128;
                    // Q: 16 dims = 8 TMEM columns per MMA, 64 columns of hi words, then 64 of lo words
#pragma unroll
                    for (int j = 0; j < 16; ++j) tc_mma_ts(tS, tmem + kTcColQ + 8 * j, dK[j & 7] + stage, idesc_s, (uint32_t)j);
                    tc_commit(s_full(b));
                    tc_commit(k_free(b));
                }
                tc_commit(s_done);
                g += it.n_steps;
            }
            tc_commit(drained);
            mbar_wait_bounded(drained, 0, p.status);
        }
        __syncwarp();
    } else {
        // ================= O issuer (warp 15): one thread issues the P V products ======================
        if (lane == 0) {
            const uint32_t idesc_o = tc_instr_desc(true);
            uint64_t dV[8];
#pragma unroll
            for (int j = 0; j < 8; ++j)  // V is [key][dim]: MN-major B operand; 64-dim halves are 16 KB apart (LBO), 8-key groups 1 KB (SBO)
                dV[j] = tc_smem_desc(smem_addr(sKV) + kTcTileBytes + j * 2048, kTcHalfBytes, 1024);
            uint32_t g = 0, m = 0;
            bool ok = true;
            for (TcItem it = get_item_1(0); it.valid && ok; it = get_item_1(++m)) {
                // the item's first product overwrites the accumulator: the previous item's rows must have been read
                if (m >= 1 && !mbar_wait_bounded(o_read, (m - 1) & 1u, p.status, p.wait_limit)) { ok = false; break; }
                for (int n = 0; n < it.n_steps; ++n) {
                    const uint32_t gn = g + n, b = gn & 1u;
                    if (!mbar_wait_bounded(v_full(b), (gn >> 1) & 1u, p.status, p.wait_limit)) { ok = false; break; }
                    if (!mbar_wait_bounded(p_full(b), (gn >> 1) & 1u, p.status, p.wait_limit)) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint64_t stage = (uint64_t)(b * (kTcStageBytes >> 4));
                    const uint32_t tP = tmem + b * 128, tO = tmem + kTcColO;
                    // P: 16 keys = 8 TMEM columns per MMA; every 32 keys hold their 16 hi words, then their 16 lo words.
                    // The accumulator carries over from tile to tile (the item's first product overwrites it).
                    tc_mma_ts(tO, tP, dV[0] + stage, idesc_o, (uint32_t)n);
#pragma unroll
                    for (int u = 1; u < 16; ++u) {
                        const int hp = u >> 3, j = u & 7;
                        tc_mma_ts(tO, tP + (j >> 1) * 32 + hp * 16 + (j & 1) * 8, dV[j] + stage, idesc_o, 1u);
                    }
                    tc_commit(o_full(b));
                    tc_commit(v_free(b));
                }
                tc_commit(o_done);
                g += it.n_steps;
            }
            // every product issued above has finished before the TMEM is released
            tc_commit(drained2);
            mbar_wait_bounded(drained2, 0, p.status);
        }
        __syncwarp();
    }
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 13) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
    }
}

}  // namespace uocr_b200
