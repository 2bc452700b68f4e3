/*
 * C ABI of the B200-native R-SWA KV-cache path (libuocr_rswa_b200.so).
 *
 * Every entry point takes plain pointers and sizes, launches hand-written sm_100a kernels on the
 * caller's stream and returns an int status (0 = ok).  Nothing here allocates device memory except
 * the explicit *_create calls; nothing synchronises the stream except the calls documented to do
 * so.  All launch entry points are safe inside CUDA-graph stream capture.
 *
 * Each declaration names the reference interface it stands in for (paths relative to the root of
 * vaachang/unlimited-ocr.cpp).  Two families exist for every operation:
 *
 *   *_f32   -- the reference's own memory layout: contiguous fp32 caches
 *              [slots][batch_cap][kv_heads*head_dim], argument lists identical to the reference's
 *              uocr::cuda::rswa_* functions plus a workspace handle where scratch is needed.
 *   *_paged -- the paged layout this library adds underneath the same semantics: a block pool of
 *              16-token blocks (bf16 or fp32 payload), a per-slot block table whose row lists the
 *              (shareable) prefix blocks first and the private ring blocks after them.
 *
 * Logical view (what parity is defined on): slot s of a sequence is prefix token s for s < P and
 * ring slot s - P otherwise; physically, token s < P lives in block table[s / 16] at offset s % 16
 * and ring slot r in block table[ceil(P / 16) + r / 16] at offset r % 16.
 */
#ifndef UOCR_RSWA_B200_H
#define UOCR_RSWA_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define UOCR_B200_API __attribute__((visibility("default")))
#else
#define UOCR_B200_API
#endif

/* A cudaStream_t, spelled without including the CUDA headers. */
typedef struct CUstream_st* uocr_b200_stream_t;

enum {
    UOCR_B200_OK = 0,
    UOCR_B200_ERR_INVALID = 1,     /* bad argument (null pointer, negative size, ...)            */
    UOCR_B200_ERR_UNSUPPORTED = 2, /* geometry outside what the kernels are built for           */
    UOCR_B200_ERR_CUDA = 3,        /* a CUDA runtime call or launch failed; see last_error()     */
    UOCR_B200_ERR_WORKSPACE = 4,   /* workspace too small for this call                          */
    UOCR_B200_ERR_NO_DEVICE = 5,   /* no usable CUDA device / not an sm_100 part                 */
    UOCR_B200_ERR_DEVICE_STATUS = 6, /* a kernel recorded a fault (bad block id, wait ran out)  */
    UOCR_B200_ERR_EXHAUSTED = 7    /* host allocator: pool exhausted                             */
};

/* KV payload types; numeric values match uocr::DType (include/uocr/common.h:17-26). */
enum { UOCR_B200_F32 = 0, UOCR_B200_BF16 = 1 };

#define UOCR_B200_BLOCK_TOKENS 16

UOCR_B200_API const char* uocr_b200_status_string(int status);
/* Message of the most recent failure on the calling thread ("" when none). */
UOCR_B200_API const char* uocr_b200_last_error(void);
/* Library / build identification, e.g. "uocr_rswa_b200 0.1 sm_100a". */
UOCR_B200_API const char* uocr_b200_version(void);
/* Number of kernels this library has launched in this process (all entry points). */
UOCR_B200_API uint64_t uocr_b200_launch_count(void);

/* ------------------------------------------------------------------------------------------------
 * Scratch for split-KV attention.  One workspace serves one stream at a time.
 * Replaces: nothing (the reference kernels need no scratch: one CTA walks a whole (query, head)
 * serially, src/kernels/cuda/rswa_attention.cu:82-148).
 * --------------------------------------------------------------------------------------------- */
typedef struct uocr_b200_workspace uocr_b200_workspace;
/* max_rows = largest number of query rows (batch, or packed prefill tokens) of any later call. */
UOCR_B200_API int uocr_b200_workspace_create(int max_rows, uocr_b200_workspace** out);
UOCR_B200_API int uocr_b200_workspace_destroy(uocr_b200_workspace* ws);
/* Synchronises `stream`, reads and clears the device status word (0 = no kernel reported a fault). */
UOCR_B200_API int uocr_b200_workspace_status(uocr_b200_workspace* ws, uocr_b200_stream_t stream,
                                             int* device_status);

/* Measurement aid: when enabled, every attention call records a CUDA event pair around its
 * partial-attention kernel on the launching stream; last_kernel_ms synchronises on the second
 * event and returns the elapsed time of the most recent call.  Keep it off inside graph capture. */
UOCR_B200_API int uocr_b200_workspace_set_timing(uocr_b200_workspace* ws, int enabled);
UOCR_B200_API int uocr_b200_workspace_last_kernel_ms(uocr_b200_workspace* ws, float* ms);

/* Output type of every attention entry point that takes this workspace (the split-KV family, the
 * fused decode steps and the tensor-core prefill): UOCR_B200_F32 (default, the reference's
 * interface) or UOCR_B200_BF16, in which case `out` is read as uint16 bf16 [rows][heads*head_dim]
 * (round-to-nearest-even on the raw bits, include/uocr/common.h:56-64) -- the input the o-projection
 * GEMM that follows the path (src/engine/gpu_decoder.cu:997) reads at half the bytes.  The setting
 * is read when a call is issued (and frozen into captured graphs). */
UOCR_B200_API int uocr_b200_workspace_set_out_dtype(uocr_b200_workspace* ws, int dtype);

/* How many polls a wait for a KV tile may take before the warp gives up (default and maximum: 2^22;
 * each poll already blocks for a hardware-defined slice).  A wait that runs out sets
 * UOCR_B200 device status bit 2 (reported by uocr_b200_workspace_status, which also clears the
 * scratch counters the abandoned launch left half-way); the warp lets its copies in flight land and
 * leaves, the kernel ends normally and the results of that launch are void.  Lowering the limit is
 * a diagnostic aid: 0 makes every wait give up at once, which exercises exactly that path without
 * hanging anything.  Applies to the split-KV attention kernels and to the tensor-core prefill
 * kernel launched with this workspace (there every role of the CTA gives up at its first wait; the
 * waits that see issued copies and tensor-core instructions through keep the full limit). */
UOCR_B200_API int uocr_b200_workspace_set_wait_limit(uocr_b200_workspace* ws, unsigned polls);

/* Opt-in launch overlap for uocr_b200_rswa_decode_step_paged calls that use this workspace.  When
 * enabled, the step is launched with programmatic stream serialization: its prologue (planning from
 * the layer's cursors, block-table reads, the first KV tiles) may run while the preceding kernel in
 * the stream is still finishing; it waits for that kernel before reading q / k / v and before
 * touching scratch.  Enable it only where the preceding kernel does not write THIS layer's cursors,
 * block table or pool (true between the layers of a decoder, whose predecessor is another layer's
 * work); leave it off otherwise, e.g. directly after a prefill of the same layer.  Default: off.
 * With overlap on, the CTAs of a launch move in as the CTAs of the preceding launch leave, so the
 * last block starts several microseconds after the rest; when every warp holds work it is given
 * 13/16 of an even share.  Results do not depend on how the work is cut. */
UOCR_B200_API int uocr_b200_workspace_set_overlap(uocr_b200_workspace* ws, int enabled);

/* Measurement aid (no reference counterpart): the rate at which this GPU streams from HBM into shared
 * memory through the path the attention kernels use -- one persistent CTA per SM, 16 warps each pulling
 * 4 KB tiles with bulk async copies, nothing written back -- in GB/s (median of 5 runs over a 1.2 GB
 * buffer read twice).  A read-only denominator to put beside a copy-bandwidth figure, which counts a
 * read and a write stream.  Allocates the buffer and synchronises: call outside stream capture. */
UOCR_B200_API int uocr_b200_workspace_stream_read_gbs(uocr_b200_workspace* ws, uocr_b200_stream_t stream, double* gbs);

/* ------------------------------------------------------------------------------------------------
 * Paged KV view of ONE layer.
 * Replaces: the per-layer buffers `batch_k_[li]`, `batch_v_[li]` + `batch_cap_` addressing
 * (src/engine/gpu_decoder.cu:904-970; base + slot*batch_cap*stride in
 * src/kernels/cuda/rswa_attention.cu:98-99,234-235,297-298,332-333).
 * --------------------------------------------------------------------------------------------- */
typedef struct {
    void* k_pool;               /* device, [num_blocks][kv_heads][16][head_dim] of dtype          */
    void* v_pool;               /* same shape                                                      */
    const int32_t* block_table; /* device, [slots][table_stride] physical block ids               */
    int32_t table_stride;
    int32_t num_blocks;
    int32_t kv_heads;
    int32_t head_dim;           /* power of two, 8..256 (bf16) or 4..256 (fp32)                    */
    int32_t dtype;              /* UOCR_B200_BF16 or UOCR_B200_F32                                 */
} uocr_b200_paged_kv;

/* ================================================================================================
 * Append (ring state machine + row write)
 * ============================================================================================= */

/* Replaces uocr::cuda::rswa_append_decode_batch (include/uocr/cuda_ops.h:95-99;
 * src/kernels/cuda/rswa_attention.cu:309-338,488-498).  Row b of k/v ([batch][kv_heads*head_dim]
 * fp32) goes to slot d_slots[b]; d_len / d_ring_pos are that layer's per-slot cursors. */
UOCR_B200_API int uocr_b200_rswa_append_decode_batch_f32(
    const float* k, const float* v, float* kcache_base, float* vcache_base, int* d_len,
    int* d_ring_pos, const int* d_prefill_len, const int* d_slots, int batch, int batch_cap,
    int window, int kv_heads, int head_dim, uocr_b200_stream_t stream);

/* Replaces uocr::cuda::rswa_append_decode (include/uocr/cuda_ops.h:84-86;
 * src/kernels/cuda/rswa_attention.cu:458-486): one cache, device cursors. */
UOCR_B200_API int uocr_b200_rswa_append_decode_f32(
    const float* k, const float* v, float* kcache, float* vcache, int* d_len, int* d_ring_pos,
    int prefill_len, int window, int kv_heads, int head_dim, uocr_b200_stream_t stream);

/* Paged form of the batched append: same cursor semantics, the row is rounded to the pool dtype
 * (bf16: nearest-even on the raw bits, include/uocr/common.h:56-64) and written through the block
 * table.  `status` may be null; otherwise out-of-range block ids are recorded there. */
UOCR_B200_API int uocr_b200_rswa_append_decode_batch_paged(
    const uocr_b200_paged_kv* kv, const float* k, const float* v, int* d_len, int* d_ring_pos,
    const int* d_prefill_len, const int* d_slots, int batch, int window,
    uocr_b200_workspace* ws, uocr_b200_stream_t stream);

/* The paged append above for ALL layers of a step in one launch.  No single reference call does this:
 * the reference appends inside its layer loop (src/engine/gpu_decoder.cu:990-993), where the K/V rows
 * of layer l+1 do not exist before layer l is done; in a decoder the append is part of the fused step
 * below.  This form is for callers that hold the rows of every layer at once -- importing a cache,
 * replaying a trace, the block-manager churn workload -- for whom `layers` launches of a few megabytes
 * each are bound by launch latency.  kv_layers[0..layers) describe pools of one geometry behind one
 * block table (1..32 layers per call); layer l reads its rows at k / v + l * kv_layer_stride (floats) and
 * its cursors at d_len / d_ring_pos + l * cursor_layer_stride (ints).  Same result as `layers` calls. */
UOCR_B200_API int uocr_b200_rswa_append_decode_batch_paged_layers(
    const uocr_b200_paged_kv* kv_layers, int layers, const float* k, const float* v, long long kv_layer_stride,
    int* d_len, int* d_ring_pos, long long cursor_layer_stride, const int* d_prefill_len, const int* d_slots,
    int batch, int window, uocr_b200_workspace* ws, uocr_b200_stream_t stream);

/* ================================================================================================
 * Prefill scatter
 * ============================================================================================= */

/* Replaces uocr::cuda::rswa_write_prefill_ragged (include/uocr/cuda_ops.h:116-119;
 * src/kernels/cuda/rswa_attention.cu:287-305,445-453): cache[d_slots[t]][d_pos[t]] <- row t. */
UOCR_B200_API int uocr_b200_rswa_write_prefill_ragged_f32(
    const float* k, const float* v, float* kcache_base, float* vcache_base, const int* d_slots,
    const int* d_pos, int total, int batch_cap, int kv_heads, int head_dim,
    uocr_b200_stream_t stream);

/* Paged form: d_pos[t] is a logical slot of the fixed region (0 <= pos < P of that slot). */
UOCR_B200_API int uocr_b200_rswa_write_prefill_ragged_paged(
    const uocr_b200_paged_kv* kv, const float* k, const float* v, const int* d_slots,
    const int* d_pos, int total, uocr_b200_workspace* ws, uocr_b200_stream_t stream);

/* Publishes the state of `n` slots in one launch.  Replaces the per-request publication after a ragged
 * prefill (src/engine/gpu_decoder.cu:1131-1150: len and ring_pos of every layer and prefill_len, one
 * blocking single-int cudaMemcpy each, 2 * layers + 1 copies per request).  d_packed holds n records of
 * 3 + table_stride int32: [slot, length, write_row, row[table_stride]]; for each record the kernel sets
 * d_len[l][slot] = length and d_ring_pos[l][slot] = 0 for every layer l (arrays laid out
 * [layers][slots]), d_prefill_len[slot] = length, and, when write_row != 0, the slot's block-table row.
 * A caller stages the records of a whole admission wave in pinned memory and brings them over with one
 * copy.  A record with length 0 and a row of -1 retires a slot: later use of it is then reported as a
 * bad block instead of touching blocks that belong to someone else.  `ws` (may be null) receives the
 * status bit for a record whose slot is out of range. */
UOCR_B200_API int uocr_b200_rswa_publish_slots(
    const int32_t* d_packed, int n, int32_t* block_table, int table_stride, int* d_len, int* d_ring_pos,
    int* d_prefill_len, int slots, int layers, uocr_b200_workspace* ws, uocr_b200_stream_t stream);

/* ================================================================================================
 * Attention.  q / out are fp32 [rows][heads*head_dim]; scale = 1/sqrt(head_dim); out = 0 for a row
 * that attends nothing.  All forms run the same split-KV kernels: a plan kernel (folded into the
 * attention kernel in the fused decode steps) and a persistent attention kernel fed by bulk async
 * copies, in which whichever warp finishes a split item last merges its partial results.
 * ============================================================================================= */

/* Replaces uocr::cuda::rswa_attention_batch (include/uocr/cuda_ops.h:104-107;
 * src/kernels/cuda/rswa_attention.cu:82-148,401-421). */
UOCR_B200_API int uocr_b200_rswa_attention_batch_f32(
    const float* q, const float* kcache_base, const float* vcache_base, const int* d_len,
    const int* d_slots, int batch, int batch_cap, int heads, int kv_heads, int head_dim, float* out,
    uocr_b200_workspace* ws, uocr_b200_stream_t stream);

UOCR_B200_API int uocr_b200_rswa_attention_batch_paged(
    const uocr_b200_paged_kv* kv, const float* q, const int* d_len, const int* d_prefill_len,
    const int* d_slots, int batch, int heads, float* out, uocr_b200_workspace* ws,
    uocr_b200_stream_t stream);

/* Replaces uocr::cuda::rswa_attention_ragged (include/uocr/cuda_ops.h:120-123;
 * src/kernels/cuda/rswa_attention.cu:218-284,423-443): packed row t attends rows [0, d_pos[t]] of
 * slot d_slots[t]. */
UOCR_B200_API int uocr_b200_rswa_attention_ragged_f32(
    const float* q, const float* kcache_base, const float* vcache_base, const int* d_slots,
    const int* d_pos, int total, int batch_cap, int heads, int kv_heads, int head_dim, float* out,
    uocr_b200_workspace* ws, uocr_b200_stream_t stream);

UOCR_B200_API int uocr_b200_rswa_attention_ragged_paged(
    const uocr_b200_paged_kv* kv, const float* q, const int* d_prefill_len, const int* d_slots,
    const int* d_pos, int total, int heads, float* out, uocr_b200_workspace* ws,
    uocr_b200_stream_t stream);

/* Replaces uocr::cuda::rswa_attention and rswa_attention_decode (include/uocr/cuda_ops.h:61-72;
 * src/kernels/cuda/rswa_attention.cu:152-214,342-379) and rswa_attention_devlen (:77-80, :381-399)
 * in one call: one cache, `seq` queries from absolute position q_start; when causal, query s sees
 * slots [0, min(len, q_start+s+1)).  The length is *d_len when d_len is non-null, else kv_len.
 * (Unlike the reference's devlen variant, any seq is handled, not just seq == 1.) */
UOCR_B200_API int uocr_b200_rswa_attention_f32(
    const float* q, const float* kcache, const float* vcache, int kv_len, const int* d_len, int seq,
    int q_start, int heads, int kv_heads, int head_dim, int causal, float* out,
    uocr_b200_workspace* ws, uocr_b200_stream_t stream);

/* Paged form for one slot: length from d_len[slot] when d_len is non-null else kv_len; the fixed
 * region length from d_prefill_len[slot] when non-null else prefill_len. */
UOCR_B200_API int uocr_b200_rswa_attention_paged(
    const uocr_b200_paged_kv* kv, int slot, const float* q, int kv_len, const int* d_len,
    int prefill_len, const int* d_prefill_len, int seq, int q_start, int heads, int causal,
    float* out, uocr_b200_workspace* ws, uocr_b200_stream_t stream);

/* Prefill of TEXT tokens over "fixed prefix + last-W window", for prompts that may be longer than
 * the window.  The reference never wraps during prefill (its whole first prefill becomes the fixed
 * region, src/engine/gpu_decoder.cu:1131-1150); this entry point implements the composition of
 * reference calls that defines the wrapped case: for each text token in order, append_decode then
 * attention(seq = 1) (src/scheduler/kv_cache.cpp:54-130).  Packed row t is text token d_pos[t] of
 * slot d_slots[t]; its K/V are first written (rounded to the pool dtype) to a caller-provided text
 * pool -- same block layout as the KV pool, `text_blocks` blocks, the request's tokens starting at
 * block d_text_block0[t] -- and the row then attends the slot's whole fixed region plus text tokens
 * (d_pos[t] - window, d_pos[t]].  Nothing is written to the KV pool; call
 * uocr_b200_rswa_ring_fill_paged afterwards. */
UOCR_B200_API int uocr_b200_rswa_prefill_text_paged(
    const uocr_b200_paged_kv* kv, void* text_k_pool, void* text_v_pool, int text_blocks,
    const float* q, const float* k, const float* v, const int* d_prefill_len, const int* d_slots,
    const int* d_pos, const int* d_text_block0, int total, int window, int heads, float* out,
    uocr_b200_workspace* ws, uocr_b200_stream_t stream);

/* Moves the last min(T, window) text tokens of every request from the text pool into its ring
 * (slot pos % window) and publishes len = P + min(T, W), ring_pos = T < W ? 0 : (T - W) % W:
 * the state T successive appends would leave.  d_text_len[t] = T of row t's request. */
UOCR_B200_API int uocr_b200_rswa_ring_fill_paged(
    const uocr_b200_paged_kv* kv, const void* text_k_pool, const void* text_v_pool, int text_blocks,
    const int* d_slots, const int* d_pos, const int* d_text_block0, const int* d_text_len,
    const int* d_prefill_len, int* d_len, int* d_ring_pos, int total, int window,
    uocr_b200_workspace* ws, uocr_b200_stream_t stream);

/* Writes packed text rows (fp32 k, v) into the text pool at token d_text_block0[t]*16 + d_pos[t],
 * rounded to the pool dtype: the first half of uocr_b200_rswa_prefill_text_paged on its own, for
 * callers that run the tensor-core attention below. */
UOCR_B200_API int uocr_b200_rswa_text_scatter_paged(
    const uocr_b200_paged_kv* kv, void* text_k_pool, void* text_v_pool, int text_blocks,
    const float* k, const float* v, const int* d_pos, const int* d_text_block0, int total,
    uocr_b200_workspace* ws, uocr_b200_stream_t stream);

/* uocr_b200_rswa_text_scatter_paged and uocr_b200_rswa_ring_fill_paged in one pass over the fp32 rows:
 * every row goes to the text pool, the last min(T, window) rows of each request also straight to
 * their ring slots, and the cursors are published -- the same final state without reading the text
 * pool back.  For callers that attend through uocr_b200_rswa_prefill_attention_tc, which reads the
 * prefix blocks and the text pool but neither the ring nor the cursors, so the call may come first. */
UOCR_B200_API int uocr_b200_rswa_text_scatter_fill_paged(
    const uocr_b200_paged_kv* kv, void* text_k_pool, void* text_v_pool, int text_blocks,
    const float* k, const float* v, const int* d_slots, const int* d_pos, const int* d_text_block0,
    const int* d_text_len, const int* d_prefill_len, int* d_len, int* d_ring_pos, int total,
    int window, uocr_b200_workspace* ws, uocr_b200_stream_t stream);

/* Ragged prefill attention on the tcgen05 tensor cores (bf16 KV, head_dim 128).  The caller
 * describes the packed query rows as tiles of at most 128 consecutive positions of one request
 * (host array, copied to the device by this call):
 *   kind 0: vision rows, causal over the slot's fixed region -- the semantics of
 *           uocr::cuda::rswa_attention_ragged (src/kernels/cuda/rswa_attention.cu:218-284);
 *   kind 1: text rows, whole fixed region + text tokens (pos - window, pos] from the text pool --
 *           the semantics of uocr_b200_rswa_prefill_text_paged.
 * K/V must already be in the pools (uocr_b200_rswa_write_prefill_ragged_paged for the fixed
 * region, uocr_b200_rswa_text_scatter_paged for the text).  Same results as the CUDA-core entry
 * points within the attention tolerance.  One persistent CTA per SM draws (tile, head) items from a
 * plan: the tiles ordered by the number of key tiles their rows see, most first.  The plan is made
 * on the device (the prefix lengths live there) by uocr_b200_rswa_prefill_plan_tc, or by this call
 * itself when h_tiles is given; with h_tiles == NULL the call reuses the workspace's last plan, which
 * must be for n_tiles tiles and this window and stays valid while the slots' prefix lengths are
 * unchanged (the layers of one forward pass share one plan).  uocr_b200_workspace_prefill_plan_serial
 * counts the plans made on a workspace, for callers that need to know theirs is still the last.
 * Planning copies the tiles from pageable host memory and the call encodes tensor maps on the host,
 * so neither can be part of a stream capture (ragged prefill shapes change from call to call
 * anyway); unwritten rows of the pools that fall into a fetched block must hold finite values (they
 * are masked, but a NaN times zero is a NaN). */
typedef struct {
    int32_t row0;   /* first packed row of the tile */
    int32_t rows;   /* 1..128 */
    int32_t slot;
    int32_t kind;   /* 0 vision / causal prefix, 1 text */
    int32_t pos0;   /* position of the first row: prefix index (kind 0) or text index (kind 1) */
    int32_t block0; /* kind 1: first block of the request in the text pool */
} uocr_b200_prefill_tile;
UOCR_B200_API int uocr_b200_rswa_prefill_attention_tc(
    const uocr_b200_paged_kv* kv, const void* text_k_pool, const void* text_v_pool, int text_blocks,
    const float* q, const int* d_prefill_len, const uocr_b200_prefill_tile* h_tiles, int n_tiles,
    int window, int heads, float* out, uocr_b200_workspace* ws, uocr_b200_stream_t stream);
UOCR_B200_API int uocr_b200_rswa_prefill_plan_tc(const uocr_b200_prefill_tile* h_tiles, int n_tiles,
                                                 const int* d_prefill_len, int window, uocr_b200_workspace* ws,
                                                 uocr_b200_stream_t stream);
UOCR_B200_API unsigned uocr_b200_workspace_prefill_plan_serial(const uocr_b200_workspace* ws);

/* One decode step of one layer in a single launch: the batched ring append of
 * uocr::cuda::rswa_append_decode_batch followed by uocr::cuda::rswa_attention_batch (the pair issued
 * at src/engine/gpu_decoder.cu:990-996), on the paged layout.  Every CTA plans from the pre-append
 * cursors, the warp that owns the tile holding a row's ring slot patches the new token into it (and
 * writes it to the pool), and the last CTA to have planned stores the new d_len / d_ring_pos (no CTA
 * reads the cursors again in that launch).  Results and final state are identical to calling the
 * two separate entry points.  batch > 1024 falls back to those two launches.  `out` may be any
 * address the device can write, pinned (device-mapped) host memory included: the kernel then
 * delivers the layer's result to the host without a copy of its own. */
UOCR_B200_API int uocr_b200_rswa_decode_step_paged(
    const uocr_b200_paged_kv* kv, const float* q, const float* k, const float* v, int* d_len,
    int* d_ring_pos, const int* d_prefill_len, const int* d_slots, int batch, int window, int heads,
    float* out, uocr_b200_workspace* ws, uocr_b200_stream_t stream);

/* The same step with the rotary embedding folded in: replaces uocr::cuda::rope followed by the two
 * calls above (src/engine/gpu_decoder.cu:988-996).  q and k are the un-rotated projections; row b is
 * rotated for position d_positions[b] exactly as src/kernels/cuda/rope_fused.cu:12-40 does (pairs
 * (i, i + head_dim/2), freq = theta^(-2i/head_dim) in fp32, angle = position * freq), q as it is
 * loaded and k before it is rounded to the pool dtype and written; v is untouched and q / k in
 * global memory are left as they are.  head_dim >= 16 (bf16) or 8 (fp32); at most 1024 rows. */
UOCR_B200_API int uocr_b200_rswa_decode_step_rope_paged(
    const uocr_b200_paged_kv* kv, const float* q, const float* k, const float* v,
    const int* d_positions, float theta, int* d_len, int* d_ring_pos, const int* d_prefill_len,
    const int* d_slots, int batch, int window, int heads, float* out, uocr_b200_workspace* ws,
    uocr_b200_stream_t stream);

/* Batched paged decode attention for callers that must not allocate.  It has no counterpart in the
 * reference.  Some hosts of this library cannot call cudaMalloc at all: an engine that hands the
 * whole GPU to its own arena at start-up (a later driver allocation fails or fragments it), a plugin
 * slot whose contract forbids allocations, or a serving loop that cannot afford the device-wide
 * synchronisation cudaMalloc/cudaFree imply.  Such a caller cannot create a uocr_b200_workspace, so
 * this variant of uocr_b200_rswa_attention_batch_paged keeps the split-KV scratch in a fixed
 * array that is part of the library image (about 2.8 MB of device memory on every GPU that loads
 * the library, held until the process exits) and allocates nothing, ever.
 *
 * Limits, checked on every call (status UOCR_B200_ERR_WORKSPACE with a message otherwise):
 * batch <= 1024 rows, head_dim <= 128, and a device of at most 160 SMs.
 *
 * The first call on a device looks up the device address of that array (a host-side query, no
 * allocation); make that first call before any stream capture begins.  All calls on one device
 * share the array: it still holds the previous call's contents when the next one starts (the call
 * clears the parts that have to start at zero itself), and two calls that overlap on the GPU --
 * different streams, or different host threads -- race on it.  Issue them on one stream, or
 * serialise them yourself.  Results are identical to the workspace-based entry point.  Arguments
 * are checked before the array is touched, so a refused call leaves it as it was. */
UOCR_B200_API int uocr_b200_rswa_attention_batch_paged_noalloc(
    const uocr_b200_paged_kv* kv, const float* q, const int* d_len, const int* d_prefill_len,
    const int* d_slots, int batch, int heads, float* out, uocr_b200_stream_t stream);

/* Device status of the allocation-free calls (no counterpart in the reference): what
 * uocr_b200_workspace_status is for workspace-based calls.  The kernels never trap on a bad block id,
 * a table row that is too short or a wait that ran out: they substitute block 0 / leave the loop and
 * set a bit of a status word that lives in the same built-in array (1 bad block id, 2 wait ran out,
 * 4 position outside the table row).  The bits accumulate over calls until this function reads them:
 * it synchronises `stream`, copies the word to *device_status (4 bytes into the caller's variable) and
 * clears it.  It allocates nothing either. */
UOCR_B200_API int uocr_b200_noalloc_status(uocr_b200_stream_t stream, int* device_status);

/* ================================================================================================
 * Block-table gather: paged storage -> the reference's logical view
 * Replaces: nothing in the reference (it has no block table, include/uocr/block_manager.h:11-13);
 * reproduces RSWACache::keys(l) / values(l) (include/uocr/kv_cache.h:64-66) for `n` slots:
 * out[i] is [capacity_rows][kv_heads*head_dim], rows >= len are zero.  out_dtype is F32 (widened)
 * or the pool dtype (raw copy).
 * ============================================================================================= */
UOCR_B200_API int uocr_b200_rswa_gather_paged(
    const uocr_b200_paged_kv* kv, const int* d_len, const int* d_prefill_len, const int* d_slots,
    int n, int capacity_rows, void* out_k, void* out_v, int out_dtype, uocr_b200_workspace* ws,
    uocr_b200_stream_t stream);

/* uocr_b200_rswa_gather_paged for ALL layers in one launch (no reference counterpart; same reason as the
 * all-layer append: retiring one sequence is `layers` launches of 10-25 MB otherwise).  Layer l reads its
 * cursors at d_len + l * cursor_layer_stride (ints) and writes its views at
 * out_k / out_v + l * out_layer_stride_bytes.  Same result as `layers` calls. */
UOCR_B200_API int uocr_b200_rswa_gather_paged_layers(
    const uocr_b200_paged_kv* kv_layers, int layers, const int* d_len, long long cursor_layer_stride,
    const int* d_prefill_len, const int* d_slots, int n, int capacity_rows, void* out_k, void* out_v,
    long long out_layer_stride_bytes, int out_dtype, uocr_b200_workspace* ws, uocr_b200_stream_t stream);

/* The same view in the layout of the reference's cache snapshots (tools/reference/export_reference.py:
 * 110-117, read back by tools/compare_reference.cpp:219-241): fp32 out[i][kv_head][s][head_dim], rows
 * at and beyond the slot's length zero-filled.  Used by the snapshot export of the host classes. */
UOCR_B200_API int uocr_b200_rswa_gather_heads_paged(
    const uocr_b200_paged_kv* kv, const int* d_len, const int* d_prefill_len, const int* d_slots,
    int n, int capacity_rows, float* out_k, float* out_v, uocr_b200_workspace* ws,
    uocr_b200_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* UOCR_RSWA_B200_H */
