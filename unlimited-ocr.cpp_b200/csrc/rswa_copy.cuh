// Memory-movement kernels of the R-SWA path: ring append (state machine + row write), ragged
// prefill scatter, and the block-table gather back to the reference's logical view.
// All are pure HBM traffic: 16-byte vector accesses, one cache row (or row chunk) per thread group.
#pragma once

#include "rswa_device.cuh"

namespace uocr_b200 {

// The ring state machine of RSWACache::append_decode (src/scheduler/kv_cache.cpp:54-82) on device
// cursors, as in rswa_append_batch_kernel (src/kernels/cuda/rswa_attention.cu:309-338) -- except
// that exactly one thread reads and updates the cursors (the reference lets every thread of the
// CTA do both without a barrier in between).  Returns the logical slot to write.
__device__ __forceinline__ int ring_advance(int* len_p, int* ring_p, int prefill_len, int window) {
    const int len = *len_p;
    int row;
    if (len < prefill_len + window) {
        row = len;
        *len_p = len + 1;
        if (len + 1 >= prefill_len + window) *ring_p = 0;
    } else {
        const int rp = *ring_p;
        row = prefill_len + rp;
        *ring_p = (rp + 1) % window;
    }
    return row;
}

// ---- contiguous fp32 caches (the reference's own layout) ----------------------------------------
__global__ void __launch_bounds__(256) rswa_append_f32_kernel(
    const float* __restrict__ k, const float* __restrict__ v, float* __restrict__ kbase,
    float* __restrict__ vbase, int* __restrict__ d_len, int* __restrict__ d_ring_pos,
    const int* __restrict__ d_prefill_len, const int* __restrict__ d_slots, int fixed_prefill,
    int batch_cap, int window, int signed_stride) {
    // signed_stride > 0: rows and bases are 16-byte aligned, copy with float4; < 0: scalar copy
    const bool vec = signed_stride > 0;
    const int stride = vec ? signed_stride : -signed_stride;
    __shared__ int s_row, s_slot;
    const int b = blockIdx.x;
    if (threadIdx.x == 0) {
        const int slot = d_slots ? d_slots[b] : 0;
        const int pfx = d_prefill_len ? d_prefill_len[slot] : fixed_prefill;
        s_row = ring_advance(d_len + slot, d_ring_pos + slot, pfx, window);
        s_slot = slot;
    }
    __syncthreads();
    const size_t dst = ((size_t)s_slot * batch_cap + s_row) * stride;
    const size_t src = (size_t)b * stride;
    if (vec) {
        const float4* k4 = reinterpret_cast<const float4*>(k + src);
        const float4* v4 = reinterpret_cast<const float4*>(v + src);
        float4* kd = reinterpret_cast<float4*>(kbase + dst);
        float4* vd = reinterpret_cast<float4*>(vbase + dst);
        for (int i = threadIdx.x; i < stride / 4; i += blockDim.x) {
            kd[i] = __ldg(k4 + i);
            vd[i] = __ldg(v4 + i);
        }
    } else {
        for (int i = threadIdx.x; i < stride; i += blockDim.x) {
            kbase[dst + i] = k[src + i];
            vbase[dst + i] = v[src + i];
        }
    }
}

__global__ void __launch_bounds__(256) rswa_scatter_f32_kernel(
    const float* __restrict__ k, const float* __restrict__ v, float* __restrict__ kbase,
    float* __restrict__ vbase, const int* __restrict__ d_slots, const int* __restrict__ d_pos,
    int batch_cap, int signed_stride) {
    const bool vec = signed_stride > 0;
    const int stride = vec ? signed_stride : -signed_stride;
    const int t = blockIdx.x;
    const size_t dst = ((size_t)d_slots[t] * batch_cap + d_pos[t]) * stride;
    const size_t src = (size_t)t * stride;
    if (vec) {
        const float4* k4 = reinterpret_cast<const float4*>(k + src);
        const float4* v4 = reinterpret_cast<const float4*>(v + src);
        float4* kd = reinterpret_cast<float4*>(kbase + dst);
        float4* vd = reinterpret_cast<float4*>(vbase + dst);
        for (int i = threadIdx.x; i < stride / 4; i += blockDim.x) {
            kd[i] = __ldg(k4 + i);
            vd[i] = __ldg(v4 + i);
        }
    } else {
        for (int i = threadIdx.x; i < stride; i += blockDim.x) {
            kbase[dst + i] = k[src + i];
            vbase[dst + i] = v[src + i];
        }
    }
}

// ---- paged pool: [block][kv_head][16][head_dim] ---------------------------------------------------
struct PagedView {
    uint8_t* k_pool;
    uint8_t* v_pool;
    const int32_t* table;
    int table_stride, num_blocks, kv_heads, head_dim;
};

// Writes one fp32 row (kv_heads*head_dim) into (block, offset) of the pool, rounding to KV.
// One thread per 16-byte destination chunk.
template <typename KV>
__device__ __forceinline__ void store_row_paged(const PagedView& pv, int blk, int off,
                                                const float* __restrict__ ksrc,
                                                const float* __restrict__ vsrc) {
    constexpr int EPC = KV::kPerChunk;
    const int hd = pv.head_dim;
    const int chunks = pv.kv_heads * hd / EPC;
    for (int c = threadIdx.x; c < chunks; c += blockDim.x) {
        const int e0 = c * EPC;
        const int head = e0 / hd, d = e0 - head * hd;
        const size_t dst = ((((size_t)blk * pv.kv_heads + head) * kBlockTokens + off) * hd + d) * KV::kBytes;
        const float4 a = __ldg(reinterpret_cast<const float4*>(ksrc + e0));
        const float4 b = __ldg(reinterpret_cast<const float4*>(vsrc + e0));
        if constexpr (EPC == 8) {
            const float4 a2 = __ldg(reinterpret_cast<const float4*>(ksrc + e0 + 4));
            const float4 b2 = __ldg(reinterpret_cast<const float4*>(vsrc + e0 + 4));
            *reinterpret_cast<uint4*>(pv.k_pool + dst) =
                make_uint4(pack_bf16x2(a.x, a.y), pack_bf16x2(a.z, a.w), pack_bf16x2(a2.x, a2.y),
                           pack_bf16x2(a2.z, a2.w));
            *reinterpret_cast<uint4*>(pv.v_pool + dst) =
                make_uint4(pack_bf16x2(b.x, b.y), pack_bf16x2(b.z, b.w), pack_bf16x2(b2.x, b2.y),
                           pack_bf16x2(b2.z, b2.w));
        } else {
            *reinterpret_cast<float4*>(pv.k_pool + dst) = a;
            *reinterpret_cast<float4*>(pv.v_pool + dst) = b;
        }
    }
}

// Pools of several layers for the kernels that serve all layers of a step in one launch (blockIdx.z = layer).
constexpr int kMaxLayersPerLaunch = 32;
struct LayerPools {
    uint8_t* k[kMaxLayersPerLaunch];
    uint8_t* v[kMaxLayersPerLaunch];
};

template <typename KV>
__device__ __forceinline__ void append_paged_row(const PagedView& pv, const float* __restrict__ k, const float* __restrict__ v,
                                                 int* __restrict__ d_len, int* __restrict__ d_ring_pos,
                                                 const int* __restrict__ d_prefill_len, const int* __restrict__ d_slots,
                                                 int window, int* __restrict__ status) {
    __shared__ int s_blk, s_off;
    const int b = blockIdx.x;
    if (threadIdx.x == 0) {
        const int slot = d_slots[b];
        const int pfx = d_prefill_len[slot];
        const int row = ring_advance(d_len + slot, d_ring_pos + slot, pfx, window);
        const int r = row - pfx;
        const int idx = (pfx + kBlockTokens - 1) / kBlockTokens + r / kBlockTokens;
        int blk = -1;
        if (r >= 0 && idx < pv.table_stride) blk = pv.table[(size_t)slot * pv.table_stride + idx];
        else if (status) atomicOr(status, kStatusBadSlot);
        if (blk < 0 || blk >= pv.num_blocks) {
            if (status) atomicOr(status, kStatusBadBlock);
            blk = -1;
        }
        s_blk = blk;
        s_off = r & (kBlockTokens - 1);
    }
    __syncthreads();
    if (s_blk < 0) return;
    const size_t src = (size_t)b * pv.kv_heads * pv.head_dim;
    store_row_paged<KV>(pv, s_blk, s_off, k + src, v + src);
}

template <typename KV>
__global__ void __launch_bounds__(256) rswa_append_paged_kernel(
    PagedView pv, const float* __restrict__ k, const float* __restrict__ v, int* __restrict__ d_len,
    int* __restrict__ d_ring_pos, const int* __restrict__ d_prefill_len,
    const int* __restrict__ d_slots, int window, int* __restrict__ status) {
    append_paged_row<KV>(pv, k, v, d_len, d_ring_pos, d_prefill_len, d_slots, window, status);
}

// The same append for every layer of a step in one launch: grid (batch, 1, layers); layer z reads its rows
// at k / v + z * kv_layer_stride and its cursors at d_len / d_ring_pos + z * cursor_layer_stride.
template <typename KV>
__global__ void __launch_bounds__(256) rswa_append_paged_layers_kernel(
    PagedView pv, const LayerPools pools, const float* __restrict__ k, const float* __restrict__ v,
    long long kv_layer_stride, int* __restrict__ d_len, int* __restrict__ d_ring_pos, long long cursor_layer_stride,
    const int* __restrict__ d_prefill_len, const int* __restrict__ d_slots, int window, int* __restrict__ status) {
    const int z = blockIdx.z;
    pv.k_pool = pools.k[z];
    pv.v_pool = pools.v[z];
    append_paged_row<KV>(pv, k + z * kv_layer_stride, v + z * kv_layer_stride, d_len + z * cursor_layer_stride,
                         d_ring_pos + z * cursor_layer_stride, d_prefill_len, d_slots, window, status);
}

template <typename KV>
__global__ void __launch_bounds__(256) rswa_scatter_paged_kernel(
    PagedView pv, const float* __restrict__ k, const float* __restrict__ v,
    const int* __restrict__ d_slots, const int* __restrict__ d_pos, int* __restrict__ status) {
    const int t = blockIdx.x;
    const int slot = d_slots[t], pos = d_pos[t];
    const int idx = pos / kBlockTokens;
    int blk = -1;
    if (pos >= 0 && idx < pv.table_stride) blk = pv.table[(size_t)slot * pv.table_stride + idx];
    if (blk < 0 || blk >= pv.num_blocks) {
        if (threadIdx.x == 0 && status) atomicOr(status, pos >= 0 && idx < pv.table_stride ? kStatusBadBlock : kStatusBadSlot);
        return;
    }
    const size_t src = (size_t)t * pv.kv_heads * pv.head_dim;
    store_row_paged<KV>(pv, blk, pos & (kBlockTokens - 1), k + src, v + src);
}

// Slot state publication: record i of `packed` is [slot, fixed-region length, write_row, row[table_stride]].
// One CTA per record stores the slot's block-table row (when write_row != 0), len = length and
// ring_pos = 0 for every layer, and prefill_len = length -- what the reference does with 2 * layers + 1
// blocking single-int copies per request after a prefill (src/engine/gpu_decoder.cu:1131-1150).
__global__ void __launch_bounds__(128) rswa_publish_slots_kernel(
    const int32_t* __restrict__ packed, int32_t* __restrict__ table, int table_stride, int* __restrict__ d_len,
    int* __restrict__ d_ring_pos, int* __restrict__ d_prefill_len, int slots, int layers, int* __restrict__ status) {
    const int32_t* rec = packed + (size_t)blockIdx.x * (3 + table_stride);
    const int slot = rec[0], length = rec[1];
    if (slot < 0 || slot >= slots || length < 0) {
        if (threadIdx.x == 0 && status) atomicOr(status, kStatusBadSlot);
        return;
    }
    if (rec[2])
        for (int i = threadIdx.x; i < table_stride; i += blockDim.x) table[(size_t)slot * table_stride + i] = rec[3 + i];
    for (int l = threadIdx.x; l < layers; l += blockDim.x) {
        d_len[(size_t)l * slots + slot] = length;
        d_ring_pos[(size_t)l * slots + slot] = 0;
    }
    if (threadIdx.x == 0) d_prefill_len[slot] = length;
}

// Text prefill scatter: packed row t (fp32) -> text pool token d_text_block0[t]*16 + d_pos[t].
template <typename KV>
__global__ void __launch_bounds__(256) rswa_scatter_text_kernel(
    PagedView text, const float* __restrict__ k, const float* __restrict__ v, const int* __restrict__ d_pos,
    const int* __restrict__ d_text_block0, int* __restrict__ status) {
    const int t = blockIdx.x;
    const int tok = d_text_block0[t] * kBlockTokens + d_pos[t];
    const int blk = tok / kBlockTokens;
    if (tok < 0 || blk >= text.num_blocks) {
        if (threadIdx.x == 0 && status) atomicOr(status, kStatusBadBlock);
        return;
    }
    const size_t src = (size_t)t * text.kv_heads * text.head_dim;
    store_row_paged<KV>(text, blk, tok & (kBlockTokens - 1), k + src, v + src);
}

// Ring fill after a text prefill: packed row t is text token d_pos[t] (of d_text_len[t] tokens) of slot
// d_slots[t]; its K/V sit in the text pool at token d_text_block0[t]*16 + d_pos[t].  The last
// min(T, window) tokens of each request are copied to ring slot (pos mod window) -- exactly where T
// successive RSWACache::append_decode calls (src/scheduler/kv_cache.cpp:54-82) leave them -- and the
// row holding the last token publishes the cursors: len = P + min(T, W), ring_pos = T < W ? 0 : (T - W) % W.
template <typename KV>
__global__ void __launch_bounds__(256) rswa_ring_fill_kernel(
    PagedView pv, const uint8_t* __restrict__ k_text, const uint8_t* __restrict__ v_text,
    const int* __restrict__ d_slots, const int* __restrict__ d_pos, const int* __restrict__ d_text_block0,
    const int* __restrict__ d_text_len, const int* __restrict__ d_prefill_len, int* __restrict__ d_len,
    int* __restrict__ d_ring_pos, int window, int* __restrict__ status) {
    constexpr int EPC = KV::kPerChunk;
    const int t = blockIdx.x;
    const int slot = d_slots[t], i = d_pos[t], T = d_text_len[t];
    const int pfx = d_prefill_len[slot];
    if (i == T - 1 && threadIdx.x == 0) {
        d_len[slot] = pfx + min(T, window);
        d_ring_pos[slot] = T < window ? 0 : (T - window) % window;
    }
    if (i < T - window) return;  // overwritten by a later token of the same request
    const int r = i % window;
    const int idx = (pfx + kBlockTokens - 1) / kBlockTokens + r / kBlockTokens;
    int blk = -1;
    if (idx < pv.table_stride) blk = pv.table[(size_t)slot * pv.table_stride + idx];
    if (blk < 0 || blk >= pv.num_blocks) {
        if (threadIdx.x == 0 && status) atomicOr(status, kStatusBadBlock);
        return;
    }
    const int src_tok = d_text_block0[t] * kBlockTokens + i;
    const int sblk = src_tok / kBlockTokens, soff = src_tok & (kBlockTokens - 1), doff = r & (kBlockTokens - 1);
    const int hd = pv.head_dim, chunks = pv.kv_heads * hd / EPC;
    for (int c = threadIdx.x; c < chunks; c += blockDim.x) {
        const int e0 = c * EPC;
        const int head = e0 / hd, d = e0 - head * hd;
        const size_t src = ((((size_t)sblk * pv.kv_heads + head) * kBlockTokens + soff) * hd + d) * KV::kBytes;
        const size_t dst = ((((size_t)blk * pv.kv_heads + head) * kBlockTokens + doff) * hd + d) * KV::kBytes;
        *reinterpret_cast<uint4*>(pv.k_pool + dst) = *reinterpret_cast<const uint4*>(k_text + src);
        *reinterpret_cast<uint4*>(pv.v_pool + dst) = *reinterpret_cast<const uint4*>(v_text + src);
    }
}

// Text scatter and ring fill in one pass over the fp32 rows: row t goes to the text pool (as
// rswa_scatter_text_kernel) and, when it is one of its request's last min(T, window) tokens, also
// straight to ring slot (pos mod window); the request's last row publishes the cursors.  Same final
// state as the two kernels above run one after the other, without reading the text pool back.
template <typename KV>
__global__ void __launch_bounds__(160) rswa_scatter_text_fill_kernel(
    PagedView pv, PagedView text, const float* __restrict__ k, const float* __restrict__ v,
    const int* __restrict__ d_slots, const int* __restrict__ d_pos, const int* __restrict__ d_text_block0,
    const int* __restrict__ d_text_len, const int* __restrict__ d_prefill_len, int* __restrict__ d_len,
    int* __restrict__ d_ring_pos, int window, int* __restrict__ status) {
    constexpr int EPC = KV::kPerChunk;
    const int t = blockIdx.x;
    const int slot = d_slots[t], i = d_pos[t], T = d_text_len[t];
    const int pfx = d_prefill_len[slot];
    if (i == T - 1 && threadIdx.x == 0) {
        d_len[slot] = pfx + min(T, window);
        d_ring_pos[slot] = T < window ? 0 : (T - window) % window;
    }
    const int tok = d_text_block0[t] * kBlockTokens + i;
    const int tblk = tok / kBlockTokens, toff = tok & (kBlockTokens - 1);
    const bool text_ok = tok >= 0 && tblk < text.num_blocks;
    int rblk = -1, roff = 0;
    if (i >= T - window) {  // not overwritten by a later token of the same request
        const int r = i % window;
        const int idx = (pfx + kBlockTokens - 1) / kBlockTokens + r / kBlockTokens;
        if (idx < pv.table_stride) rblk = pv.table[(size_t)slot * pv.table_stride + idx];
        if (rblk < 0 || rblk >= pv.num_blocks) {
            if (threadIdx.x == 0 && status) atomicOr(status, kStatusBadBlock);
            rblk = -1;
        }
        roff = r & (kBlockTokens - 1);
    }
    if (!text_ok && threadIdx.x == 0 && status) atomicOr(status, kStatusBadBlock);
    const int hd = pv.head_dim, chunks = pv.kv_heads * hd / EPC;
    const float* ksrc = k + (size_t)t * pv.kv_heads * hd;
    const float* vsrc = v + (size_t)t * pv.kv_heads * hd;
    for (int c = threadIdx.x; c < chunks; c += blockDim.x) {
        const int e0 = c * EPC;
        const int head = e0 / hd, d = e0 - head * hd;
        uint4 kw, vw;
        const float4 a = __ldg(reinterpret_cast<const float4*>(ksrc + e0));
        const float4 b = __ldg(reinterpret_cast<const float4*>(vsrc + e0));
        if constexpr (EPC == 8) {
            const float4 a2 = __ldg(reinterpret_cast<const float4*>(ksrc + e0 + 4));
            const float4 b2 = __ldg(reinterpret_cast<const float4*>(vsrc + e0 + 4));
            kw = make_uint4(pack_bf16x2(a.x, a.y), pack_bf16x2(a.z, a.w), pack_bf16x2(a2.x, a2.y), pack_bf16x2(a2.z, a2.w));
            vw = make_uint4(pack_bf16x2(b.x, b.y), pack_bf16x2(b.z, b.w), pack_bf16x2(b2.x, b2.y), pack_bf16x2(b2.z, b2.w));
        } else {
            kw = make_uint4(__float_as_uint(a.x), __float_as_uint(a.y), __float_as_uint(a.z), __float_as_uint(a.w));
            vw = make_uint4(__float_as_uint(b.x), __float_as_uint(b.y), __float_as_uint(b.z), __float_as_uint(b.w));
        }
        if (text_ok) {
            const size_t dst = ((((size_t)tblk * pv.kv_heads + head) * kBlockTokens + toff) * hd + d) * KV::kBytes;
            *reinterpret_cast<uint4*>(text.k_pool + dst) = kw;
            *reinterpret_cast<uint4*>(text.v_pool + dst) = vw;
        }
        if (rblk >= 0) {
            const size_t dst = ((((size_t)rblk * pv.kv_heads + head) * kBlockTokens + roff) * hd + d) * KV::kBytes;
            *reinterpret_cast<uint4*>(pv.k_pool + dst) = kw;
            *reinterpret_cast<uint4*>(pv.v_pool + dst) = vw;
        }
    }
}

// Gather: logical row s of slot d_slots[i] -> out[i][s][:]; rows >= len are zero-filled.
// HEAD_MAJOR: out[i][head][s][:] instead (the layout of the reference's exported cache snapshots).
// grid = (capacity_rows, n); one thread per 16-byte pool chunk.
template <typename KV, bool WIDEN, bool HEAD_MAJOR>
__device__ __forceinline__ void gather_paged_row(const PagedView& pv, const int* __restrict__ d_len,
                                                 const int* __restrict__ d_prefill_len, const int* __restrict__ d_slots,
                                                 int capacity_rows, uint8_t* __restrict__ out_k, uint8_t* __restrict__ out_v,
                                                 int* __restrict__ status) {
    constexpr int EPC = KV::kPerChunk;
    constexpr int OUT_B = WIDEN ? 4 : KV::kBytes;
    const int s = blockIdx.x, i = blockIdx.y;
    const int slot = d_slots[i];
    const int len = d_len[slot], pfx = d_prefill_len[slot];
    const int hd = pv.head_dim, row_elems = pv.kv_heads * hd;
    const size_t out_row = ((size_t)i * capacity_rows + s) * row_elems * OUT_B;
    const int chunks = row_elems / EPC;
    int blk = -1, off = 0;
    if (s < len) {
        int idx;
        if (s < pfx) {
            idx = s / kBlockTokens;
            off = s & (kBlockTokens - 1);
        } else {
            const int r = s - pfx;
            idx = (pfx + kBlockTokens - 1) / kBlockTokens + r / kBlockTokens;
            off = r & (kBlockTokens - 1);
        }
        if (idx < pv.table_stride) blk = pv.table[(size_t)slot * pv.table_stride + idx];
        if (blk < 0 || blk >= pv.num_blocks) {
            if (threadIdx.x == 0 && status) atomicOr(status, kStatusBadBlock);
            blk = -1;
        }
    }
    for (int c = threadIdx.x; c < chunks; c += blockDim.x) {
        const int e0 = c * EPC;
        const int head = e0 / hd, d = e0 - head * hd;
        uint4 kw = make_uint4(0, 0, 0, 0), vw = kw;
        if (blk >= 0) {
            const size_t src = ((((size_t)blk * pv.kv_heads + head) * kBlockTokens + off) * hd + d) * KV::kBytes;
            kw = *reinterpret_cast<const uint4*>(pv.k_pool + src);
            vw = *reinterpret_cast<const uint4*>(pv.v_pool + src);
        }
        const size_t dst = HEAD_MAJOR ? ((((size_t)i * pv.kv_heads + head) * capacity_rows + s) * hd + d) * OUT_B
                                      : out_row + (size_t)e0 * OUT_B;
        if constexpr (WIDEN && EPC == 8) {
            float4* ko = reinterpret_cast<float4*>(out_k + dst);
            float4* vo = reinterpret_cast<float4*>(out_v + dst);
            ko[0] = make_float4(bf16_lo(kw.x), bf16_hi(kw.x), bf16_lo(kw.y), bf16_hi(kw.y));
            ko[1] = make_float4(bf16_lo(kw.z), bf16_hi(kw.z), bf16_lo(kw.w), bf16_hi(kw.w));
            vo[0] = make_float4(bf16_lo(vw.x), bf16_hi(vw.x), bf16_lo(vw.y), bf16_hi(vw.y));
            vo[1] = make_float4(bf16_lo(vw.z), bf16_hi(vw.z), bf16_lo(vw.w), bf16_hi(vw.w));
        } else {
            *reinterpret_cast<uint4*>(out_k + dst) = kw;
            *reinterpret_cast<uint4*>(out_v + dst) = vw;
        }
    }
}

template <typename KV, bool WIDEN, bool HEAD_MAJOR = false>
__global__ void __launch_bounds__(256) rswa_gather_paged_kernel(
    PagedView pv, const int* __restrict__ d_len, const int* __restrict__ d_prefill_len,
    const int* __restrict__ d_slots, int capacity_rows, uint8_t* __restrict__ out_k,
    uint8_t* __restrict__ out_v, int* __restrict__ status) {
    gather_paged_row<KV, WIDEN, HEAD_MAJOR>(pv, d_len, d_prefill_len, d_slots, capacity_rows, out_k, out_v, status);
}

// The same gather for every layer in one launch: grid (capacity_rows, n, layers); layer z reads its cursors at
// d_len + z * cursor_layer_stride and writes its views at out_k / out_v + z * out_layer_stride_bytes.
template <typename KV, bool WIDEN>
__global__ void __launch_bounds__(256) rswa_gather_paged_layers_kernel(
    PagedView pv, const LayerPools pools, const int* __restrict__ d_len, long long cursor_layer_stride,
    const int* __restrict__ d_prefill_len, const int* __restrict__ d_slots, int capacity_rows,
    uint8_t* __restrict__ out_k, uint8_t* __restrict__ out_v, long long out_layer_stride_bytes, int* __restrict__ status) {
    const int z = blockIdx.z;
    pv.k_pool = pools.k[z];
    pv.v_pool = pools.v[z];
    gather_paged_row<KV, WIDEN, false>(pv, d_len + z * cursor_layer_stride, d_prefill_len, d_slots, capacity_rows,
                                       out_k + z * out_layer_stride_bytes, out_v + z * out_layer_stride_bytes, status);
}

}  // namespace uocr_b200
