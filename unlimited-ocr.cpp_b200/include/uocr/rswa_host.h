// Host-side C++17 mirror of the reference's R-SWA interfaces, backed by libuocr_rswa_b200.so.
//
// Same namespace, class names, method names, argument meaning and error behaviour as
// vaachang/unlimited-ocr.cpp, so its callers and its own unit tests compile against these headers
// unchanged:
//
//   uocr::Error, UOCR_CHECK                    include/uocr/common.h:33-43
//   uocr::MemoryPool                           include/uocr/memory_pool.h:16-51
//   uocr::PrefixEntry, uocr::BlockManager      include/uocr/block_manager.h:25-79
//   uocr::ReqState/Request/Batch/
//         ContinuousBatchScheduler             include/uocr/continuous_batch.h:21-104
//   uocr::RSWACache                            include/uocr/kv_cache.h:23-86
//   uocr::cuda::GpuRSWACache                   include/uocr/gpu_cache.h:21-72
//   uocr::cuda::rswa_* free functions          include/uocr/cuda_ops.h:59-123
//
// What differs underneath: the KV of RSWACache / GpuRSWACache lives on the GPU in paged 16-token
// blocks (block table + device cursors) and every operation is a kernel launch through the C ABI;
// host pointers returned by keys()/values() are a mirror filled on demand by the block-table gather.
// New on top of the reference surface: uocr::cuda::PagedBatchKV (the batch KV state that the
// reference keeps inside GpuDecoder, src/engine/gpu_decoder.cu:904-970, gpu_decoder.h:246-258) and
// uocr::SlotAllocator (the slot free-list of Engine::generate_batch, src/engine/engine.cpp:306-318).
#pragma once

#include <cstddef>
#include <cstdint>
#include <deque>
#include <memory>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

#include "uocr_rswa_b200.h"

#if defined(__GNUC__)
#define UOCR_HOST_API __attribute__((visibility("default")))
#else
#define UOCR_HOST_API
#endif

typedef struct CUstream_st* cudaStream_t;  // same type the CUDA runtime headers declare

namespace uocr {

using i32 = std::int32_t;
using i64 = std::int64_t;
using u32 = std::uint32_t;
using u64 = std::uint64_t;

enum class DType : std::uint8_t { F32 = 0, BF16 = 1, F16 = 2, I32 = 3, I8 = 4, U8 = 5, I4 = 6, U4 = 7 };

// Exception carrying file:line, thrown by every host-side precondition check.
class UOCR_HOST_API Error : public std::runtime_error {
public:
    Error(const std::string& what, const char* file, int line)
        : std::runtime_error(std::string(file) + ":" + std::to_string(line) + ": " + what) {}
};

#define UOCR_THROW(msg) throw ::uocr::Error((msg), __FILE__, __LINE__)
#define UOCR_CHECK(cond, msg)         \
    do {                              \
        if (!(cond)) UOCR_THROW(msg); \
    } while (0)

// bf16 <-> fp32 on raw bits (round to nearest even; NaN not special-cased), as common.h:49-64.
inline float bf16_to_f32(std::uint16_t h) {
    const u32 bits = static_cast<u32>(h) << 16;
    float f;
    __builtin_memcpy(&f, &bits, sizeof f);
    return f;
}
inline std::uint16_t f32_to_bf16(float f) {
    u32 bits;
    __builtin_memcpy(&bits, &f, sizeof bits);
    bits += 0x7fffu + ((bits >> 16) & 1u);
    return static_cast<std::uint16_t>(bits >> 16);
}

// ------------------------------------------------------------------------------------------------
// Offset arena: first fit over an offset-ordered free list, alignment padding and tail returned to
// the list, `used` counts padding, free() coalesces with both neighbours.
// ------------------------------------------------------------------------------------------------
class UOCR_HOST_API MemoryPool {
public:
    struct Block {
        std::size_t offset = 0;
        std::size_t size = 0;
    };

    explicit MemoryPool(std::size_t bytes = 0, std::size_t alignment = 256);

    void reserve(std::size_t bytes);
    void reset();
    i64 allocate(std::size_t bytes, std::size_t alignment = 0);  // offset, or -1
    void free(i64 offset, std::size_t bytes);

    std::size_t total() const { return total_; }
    std::size_t used() const { return used_; }
    std::size_t peak() const { return peak_; }
    std::size_t alignment() const { return alignment_; }
    double fragmentation() const;
    std::size_t num_free_blocks() const { return spans_.size(); }

    // The reference backs the arena with host bytes; here they are materialised on first use only
    // (the KV itself never lives in the arena, it is bookkeeping in both code bases).
    std::uint8_t* base();
    const std::uint8_t* base() const;

private:
    std::size_t total_ = 0, used_ = 0, peak_ = 0, alignment_ = 256;
    std::vector<Block> spans_;  // free spans, ascending offset
    mutable std::vector<std::uint8_t> backing_;
};

struct PrefixEntry {
    std::string key;
    int prefill_len = 0;
    std::size_t bytes = 0;
    int refcount = 0;
    i64 offset = -1;
};

class UOCR_HOST_API BlockManager {
public:
    BlockManager(std::size_t prefix_pool_bytes, std::size_t ring_pool_bytes);

    PrefixEntry* acquire_prefix(const std::string& key, int prefill_len, std::size_t bytes);
    void release_prefix(const std::string& key);
    i64 allocate_ring(std::size_t bytes);
    void free_ring(i64 offset, std::size_t bytes);

    std::size_t live_prefixes() const { return table_.size(); }
    std::size_t total_prefix_bytes() const;
    std::size_t shared_prefix_bytes() const { return shared_now_; }
    std::size_t peak_prefix_bytes() const { return shared_peak_; }
    const MemoryPool& prefix_pool() const { return prefix_arena_; }
    const MemoryPool& ring_pool() const { return ring_arena_; }

    struct Stats {
        std::size_t prefix_live_bytes = 0;
        std::size_t prefix_peak_bytes = 0;
        std::size_t prefix_shared_bytes = 0;
        std::size_t ring_live_bytes = 0;
        std::size_t ring_peak_bytes = 0;
        double prefix_fragmentation = 0.0;
        double ring_fragmentation = 0.0;
        std::size_t live_prefixes = 0;
    };
    Stats stats() const;

private:
    void refresh_shared();
    MemoryPool prefix_arena_, ring_arena_;
    std::unordered_map<std::string, PrefixEntry> table_;
    std::size_t shared_now_ = 0, shared_peak_ = 0;
};

class RSWACache;

enum class ReqState { Waiting, Prefilling, Decoding, Finished };

struct Request {
    int id = -1;
    std::string doc_key;
    std::vector<int> prompt_tokens;
    std::vector<int> output_tokens;
    ReqState state = ReqState::Waiting;
    int max_new_tokens = 4096;
    bool stopped = false;
    std::shared_ptr<RSWACache> cache;
    double arrival_time = 0.0, prefill_time = 0.0, first_token_time = 0.0, finish_time = 0.0;
    int decode_steps = 0;

    bool is_finished() const { return state == ReqState::Finished; }
    int seq_len() const { return static_cast<int>(prompt_tokens.size() + output_tokens.size()); }
};

struct Batch {
    std::vector<int> prefill;
    std::vector<int> decode;
    bool empty() const { return prefill.empty() && decode.empty(); }
};

class UOCR_HOST_API ContinuousBatchScheduler {
public:
    struct Stats {
        std::uint64_t total_requests = 0, finished_requests = 0, prefill_tokens = 0, decode_tokens = 0;
        std::size_t waiting = 0, running = 0;
        double last_batch_size = 0.0;
    };

    explicit ContinuousBatchScheduler(int max_batch_size = 16, int min_batch_size = 4)
        : max_batch_(max_batch_size), min_batch_(min_batch_size) {}

    int add_request(Request r);
    Batch build_batch();
    void mark_prefilled(int id);
    void mark_prefilling(int id);
    bool add_token(int id, int token);
    void finish(int id);
    Request* get(int id);
    const Request* get(int id) const;

    bool empty() const { return all_.empty(); }
    bool has_work() const { return !queue_.empty() || !active_.empty(); }
    int max_batch_size() const { return max_batch_; }
    int min_batch_size() const { return min_batch_; }
    void set_max_batch_size(int v) { max_batch_ = v; }
    void set_min_batch_size(int v) { min_batch_ = v; }
    Stats stats() const;
    const std::vector<int>& running() const { return active_; }

private:
    int max_batch_, min_batch_;
    int next_id_ = 0;
    std::deque<int> queue_;
    std::vector<int> active_;
    std::unordered_map<int, Request> all_;
};

// Slot free-list of the batch loop: slots are handed out from the back (so the first admissions get
// the highest numbers) and a released slot is the next one reused (src/engine/engine.cpp:306-318,341-347).
class UOCR_HOST_API SlotAllocator {
public:
    explicit SlotAllocator(int slots = 0) { reset(slots); }
    void reset(int slots);
    int acquire(int request_id);  // throws "no free slot" when exhausted
    void release(int request_id);
    int slot_of(int request_id) const;  // -1 when unknown
    int free_count() const { return static_cast<int>(free_.size()); }

private:
    std::vector<int> free_;
    std::unordered_map<int, int> by_request_;
};

namespace detail {
class PagedSeqStore;  // one sequence, all layers, on the device
}

// ------------------------------------------------------------------------------------------------
// RSWACache: host-pointer interface of the reference, KV held on the GPU.
// ------------------------------------------------------------------------------------------------
class UOCR_HOST_API RSWACache {
public:
    RSWACache();
    RSWACache(int num_layers, int kv_heads, int head_dim, int window);
    ~RSWACache();
    RSWACache(RSWACache&&) noexcept;
    RSWACache& operator=(RSWACache&&) noexcept;
    RSWACache(const RSWACache&) = delete;
    RSWACache& operator=(const RSWACache&) = delete;

    void configure(int num_layers, int kv_heads, int head_dim, int window);
    // Extension: choose the device payload type before reset() (default F32, which keeps the
    // reference's bit-exact fp32 contents; BF16 halves the bytes and rounds on append).
    void set_kv_dtype(DType t);
    void reset(int prefill_len);

    int num_layers() const;
    int kv_heads() const;
    int head_dim() const;
    int window() const;
    int prefill_len() const;
    int length(int layer) const;
    int ring_pos(int layer) const;
    bool ring_started(int layer) const;
    int capacity() const;

    void write_prefill(int layer, const float* k, const float* v, int seq);
    void append_decode(int layer, const float* k, const float* v);
    void attention(int layer, const float* q, int seq, int q_start, float* out, int heads, bool causal) const;

    int len(int layer) const { return length(layer); }
    const float* keys(int layer) const;
    const float* values(int layer) const;
    float* mutable_keys(int layer);
    float* mutable_values(int layer);
    std::size_t bytes() const;

private:
    std::unique_ptr<detail::PagedSeqStore> s_;
};

namespace cuda {

// Device-pointer interface of the reference's single-request GPU cache.
class UOCR_HOST_API GpuRSWACache {
public:
    GpuRSWACache();
    GpuRSWACache(int num_layers, int kv_heads, int head_dim, int window);
    ~GpuRSWACache();
    GpuRSWACache(const GpuRSWACache&) = delete;
    GpuRSWACache& operator=(const GpuRSWACache&) = delete;

    void configure(int num_layers, int kv_heads, int head_dim, int window);
    void set_kv_dtype(DType t);
    void reset(int prefill_len);
    void write_prefill(int layer, const float* d_k, const float* d_v, int seq, cudaStream_t stream = nullptr);
    void append_decode(int layer, const float* d_k, const float* d_v, cudaStream_t stream = nullptr);
    void reset_device_state(int prefill_len, cudaStream_t stream = nullptr);
    void append_decode_device(int layer, const float* d_k, const float* d_v, cudaStream_t stream = nullptr);
    const int* len_dev(int layer) const;
    // Attention over the length this object's HOST cursor holds (the reference's host-cursor path,
    // src/kernels/cuda/gpu_cache.cu:141-145).  The length is frozen into the launch: inside a captured
    // graph use attention_devlen instead.
    void attention(int layer, const float* d_q, int seq, int q_start, float* d_out, int heads, bool causal,
                   cudaStream_t stream = nullptr) const;
    // Attention over the DEVICE length len_dev(layer): the call to pair with append_decode_device inside a
    // captured decode graph.  It stands in for the reference's graph call site, which passes
    // keys(layer) / values(layer) and len_dev(layer) to rswa_attention_devlen
    // (src/engine/gpu_decoder.cu:502-505): here the cache is paged, so the attention reads the blocks
    // directly instead of a contiguous view, and a replayed graph sees every appended token.
    void attention_devlen(int layer, const float* d_q, int seq, int q_start, float* d_out, int heads, bool causal,
                          cudaStream_t stream = nullptr) const;

    int len(int layer) const;
    int prefill_len() const;
    int window() const;
    int capacity() const;
    int num_layers() const;
    // Device pointers to the logical fp32 view [capacity][kv_heads*head_dim]: a SNAPSHOT made by a
    // block-table gather launched on `stream` when the call is made, valid until the next call on this
    // object.  Not for use inside stream capture (a replayed graph would attend over the snapshot taken
    // at capture time): the call throws uocr::Error when `stream` is capturing.
    const float* keys(int layer, cudaStream_t stream = nullptr) const;
    const float* values(int layer, cudaStream_t stream = nullptr) const;

private:
    std::unique_ptr<detail::PagedSeqStore> s_;
};

// The reference's eight R-SWA entry points, same signatures (contiguous fp32 caches).  The reference's
// kernels need no scratch; the split-KV kernels here do, and the attention wrappers take it from a
// workspace kept per (device, stream): two streams never share scratch, and a workspace, once handed to
// a launch, is never freed or moved (a captured graph keeps pointing into it).  rswa_prepare creates the
// workspace of a stream for up to `max_rows` query rows per call (packed prefill tokens or batch rows);
// without it the first attention call on a stream prepares 4096 rows itself, which allocates and so must
// not happen inside stream capture -- a call that finds no workspace while its stream is capturing, or
// that has more rows than were prepared, launches nothing and reports the error on stderr like the
// reference's wrappers do for CUDA errors.  A later rswa_prepare with a larger count adds a larger
// workspace for subsequent calls and leaves the old one in place.  Returns false when it failed.
UOCR_HOST_API bool rswa_prepare(cudaStream_t stream, int max_rows);
UOCR_HOST_API void rswa_attention_decode(const float* q, const float* kcache, const float* vcache, int kv_len,
                                         int heads, int kv_heads, int head_dim, float* out, cudaStream_t stream = nullptr);
UOCR_HOST_API void rswa_attention(const float* q, const float* kcache, const float* vcache, int kv_len, int seq,
                                  int q_start, int heads, int kv_heads, int head_dim, bool causal, float* out,
                                  cudaStream_t stream = nullptr);
UOCR_HOST_API void rswa_attention_devlen(const float* q, const float* kcache, const float* vcache, const int* d_len,
                                         int seq, int q_start, int heads, int kv_heads, int head_dim, bool causal,
                                         float* out, cudaStream_t stream = nullptr);
UOCR_HOST_API void rswa_append_decode(const float* k, const float* v, float* kcache, float* vcache, int* d_len,
                                      int* d_ring_pos, int prefill_len, int window, int kv_heads, int head_dim,
                                      cudaStream_t stream = nullptr);
UOCR_HOST_API void rswa_append_decode_batch(const float* k, const float* v, float* kcache_base, float* vcache_base,
                                            int* d_len, int* d_ring_pos, const int* d_prefill_len, const int* d_slots,
                                            int batch, int batch_cap, int window, int kv_heads, int head_dim,
                                            cudaStream_t stream = nullptr);
UOCR_HOST_API void rswa_attention_batch(const float* q, const float* kcache_base, const float* vcache_base,
                                        const int* d_len, const int* d_slots, int batch, int batch_cap, int heads,
                                        int kv_heads, int head_dim, float* out, cudaStream_t stream = nullptr);
UOCR_HOST_API void rswa_write_prefill_ragged(const float* k, const float* v, float* kcache_base, float* vcache_base,
                                             const int* d_slots, const int* d_pos, int total, int batch_cap,
                                             int kv_heads, int head_dim, cudaStream_t stream = nullptr);
UOCR_HOST_API void rswa_attention_ragged(const float* q, const float* kcache_base, const float* vcache_base,
                                         const int* d_slots, const int* d_pos, int total, int batch_cap, int heads,
                                         int kv_heads, int head_dim, float* out, cudaStream_t stream = nullptr);

// ------------------------------------------------------------------------------------------------
// PagedBatchKV: the batch KV state of the decoder (what GpuDecoder::batch_configure allocates and
// attention_block_batch / attention_block_ragged drive), on the paged pool with physically shared
// prefixes.  Block ids come from a BlockManager run in block units (1 block == 256 arena bytes).
// ------------------------------------------------------------------------------------------------
class UOCR_HOST_API PagedBatchKV {
public:
    struct Config {
        int slots = 0, layers = 0, kv_heads = 0, head_dim = 0, window = 0;
        int max_prefix_tokens = 0;     // longest fixed region a slot may have
        int prefix_arena_blocks = 0;   // block ids [0, prefix_arena_blocks)
        int ring_arena_blocks = 0;     // block ids [prefix_arena_blocks, +ring_arena_blocks)
        DType dtype = DType::BF16;
    };
    struct Admission {
        int slot = -1;
        bool prefix_is_new = false;  // true: the caller must prefill the prefix through this slot
        int prefix_refcount = 0;
    };

    PagedBatchKV();
    ~PagedBatchKV();
    PagedBatchKV(const PagedBatchKV&) = delete;
    PagedBatchKV& operator=(const PagedBatchKV&) = delete;

    // Reuses the allocation when the shape is unchanged (only state is cleared), like the reference's
    // batch_configure; otherwise reallocates -- captured graphs must then be dropped by the caller.
    // Returns true when buffers were (re)allocated.
    bool configure(const Config& cfg);
    const Config& config() const;

    // Binds a slot to a document prefix (shared by doc_key, refcounted) and a private ring and publishes
    // its table row, len = P, ring_pos = 0 and prefill = P for every layer.
    Admission admit(int slot, const std::string& doc_key, int prefix_len, cudaStream_t stream = nullptr);
    // A whole admission wave at once: the table rows and cursors of every admitted slot are staged in one
    // pinned buffer, brought over by ONE copy and applied by one kernel on `stream`; no host
    // synchronisation (the staging buffers alternate and are guarded by events).  Replaces the
    // 2 * layers + 1 blocking copies per request of src/engine/gpu_decoder.cu:1131-1150.  All-or-nothing:
    // if a request cannot be placed (arena exhausted) the earlier ones of the wave are rolled back and
    // the call throws.
    struct WaveItem {
        int slot = -1;
        std::string doc_key;
        int prefix_len = 0;
    };
    std::vector<Admission> admit_wave(const std::vector<WaveItem>& items, cudaStream_t stream = nullptr);
    // Frees the ring and drops the prefix reference.  The slot's device table row is overwritten with -1
    // and its cursors with 0 by a kernel queued on `stream`, so a stale use of the slot is reported as a bad
    // block instead of touching blocks that may already belong to another sequence.  Ordering is the
    // caller's: issue the release on the stream that carried the slot's last launch (the blocks may be
    // handed out again by the next admit, whose own writes are queued behind the release on that stream),
    // and drop or re-stage captured graphs whose row -> slot map still names the slot.
    void release(int slot, cudaStream_t stream = nullptr);
    // Engine-style state publication after a ragged prefill (src/engine/gpu_decoder.cu:1131-1150).
    void publish_prefill_state(int slot, int prefix_len, cudaStream_t stream = nullptr);
    // Launch overlap between the fused steps of consecutive layers (uocr_b200_workspace_set_overlap).
    void set_overlap(bool enabled);

    // The decode step of all layers as one CUDA graph per batch size, as GpuDecoder::capture_batch_graph /
    // batch_decode keep one per observed batch size (src/engine/gpu_decoder.cu:746-772,1210-1213).  The
    // graph holds layers x decode_step (or decode_step_rope when d_positions is set) on FIXED buffers: layer l
    // reads q + l * q_layer_stride, k / v + l * kv_layer_stride and writes out + l * out_layer_stride
    // (strides in floats); d_slots (and d_positions) are device arrays the caller refreshes before a replay.
    // capture_step returns true when it captured (false: a graph for this batch size and these buffers
    // exists already); graphs are dropped when configure() reallocates, as the reference invalidates its
    // batch graphs (:929-931).  Cursors live on the device, so one graph replays across the warm-up ->
    // ring boundary.
    struct StepIO {
        const float* q = nullptr;
        const float* k = nullptr;
        const float* v = nullptr;
        float* out = nullptr;
        long long q_layer_stride = 0, kv_layer_stride = 0, out_layer_stride = 0;
        const int* d_slots = nullptr;
        int heads = 0;
        const int* d_positions = nullptr;  // non-null: rotary embedding folded into the step
        float rope_theta = 10000.f;
    };
    bool capture_step(int batch, const StepIO& io, cudaStream_t stream);
    void replay_step(int batch, cudaStream_t stream);
    int step_graph_count() const;
    void drop_step_graphs();

    // Per-layer calls; every pointer is a device pointer, d_slots maps batch rows to slots.
    void append_decode_batch(int layer, const float* k, const float* v, const int* d_slots, int batch,
                             cudaStream_t stream = nullptr);
    void attention_batch(int layer, const float* q, const int* d_slots, int batch, int heads, float* out,
                         cudaStream_t stream = nullptr);
    void decode_step(int layer, const float* q, const float* k, const float* v, const int* d_slots, int batch,
                     int heads, float* out, cudaStream_t stream = nullptr);
    // decode_step with uocr::cuda::rope folded in: q and k are the un-rotated projections, d_positions[b]
    // the position of batch row b (src/engine/gpu_decoder.cu:988-996 in one launch).
    void decode_step_rope(int layer, const float* q, const float* k, const float* v, const int* d_positions, float theta,
                          const int* d_slots, int batch, int heads, float* out, cudaStream_t stream = nullptr);
    void write_prefill_ragged(int layer, const float* k, const float* v, const int* d_row_slots, const int* d_pos,
                              int total, cudaStream_t stream = nullptr);
    void attention_ragged(int layer, const float* q, const int* d_row_slots, const int* d_pos, int total, int heads,
                          float* out, cudaStream_t stream = nullptr);
    // Windowed ragged prefill, for prompts that may be longer than the window: the prefix is the vision
    // part, text tokens attend prefix + the last `window` text tokens, and the ring and cursors end up as
    // text_rows successive append_decode calls would leave them (src/scheduler/kv_cache.cpp:54-130 by
    // composition).  Packed row order of q / k / v / out: the vision rows of every request, in request
    // order, then the text rows of every request.
    struct WindowedPrefill {
        int slot = -1;
        int vision_rows = 0;  // the slot's prefix length, or 0 when the (shared) prefix is already resident
        int text_rows = 0;
    };
    // Builds and uploads the row index arrays and the query-tile list and grows the text pool when it is
    // too small (allocates and synchronises: call outside stream capture).  Returns the packed row count.
    int plan_windowed_prefill(const std::vector<WindowedPrefill>& requests, cudaStream_t stream = nullptr);
    // One layer of the planned prefill: scatter of K/V (prefix blocks; text pool), attention, ring fill and
    // cursor publication.  bf16 KV with head_dim 128 runs on the tensor cores, everything else on CUDA cores.
    void windowed_prefill_layer(int layer, const float* q, const float* k, const float* v, int heads, float* out,
                                cudaStream_t stream = nullptr);

    // Logical fp32 view of `n` slots: out[i] is [max_prefix_tokens + window][kv_heads*head_dim].
    void gather(int layer, const int* d_slots, int n, float* out_k, float* out_v, cudaStream_t stream = nullptr);

    // Cache snapshot of one slot in the reference's on-disk alignment format (written by
    // tools/reference/export_reference.py:21-26,110-117,155-160; read by tools/compare_reference.cpp:25-36,
    // 219-241): per layer `<tag>_k_<l>.bin` and `<tag>_v_<l>.bin`, raw little-endian fp32 of shape
    // [kv_heads, len, head_dim] (logical slot order: prefix, then ring slots), and `manifest.json` with
    // one {"file","shape","dtype":"<f4"} entry per tensor plus "window", "cache_layers", "kv_heads",
    // "head_dim" and "<tag>_cache_len".  tag is "prefill" or "final"; a second call with another tag into
    // the same directory extends the manifest.  Synchronises the stream and writes files: not capturable.
    void export_snapshot(const std::string& dir, int slot, const std::string& tag, cudaStream_t stream = nullptr);

    const BlockManager& blocks() const;
    const std::vector<int>& table_row(int slot) const;  // host copy of the slot's block ids (-1 = unused)
    int device_status(cudaStream_t stream = nullptr);   // synchronises; 0 = no kernel recorded a fault
    const uocr_b200_paged_kv& layer_view(int layer) const;
    int* d_len(int layer) const;
    int* d_ring_pos(int layer) const;
    int* d_prefill_len() const;

private:
    struct Impl;
    std::unique_ptr<Impl> p_;
};

// ------------------------------------------------------------------------------------------------
// GpuDecoderKV: the KV half of GpuDecoder's continuous-batching interface under the reference's own
// method names (include/uocr/gpu_decoder.h:69-87, src/engine/gpu_decoder.cu:904-1213), over a
// PagedBatchKV.  A decoder keeps its projections, rotary embedding, MoE and lm_head and replaces the
// KV members (gpu_decoder.h:246-258) and the three attention call sites by calls on this object:
//
//   batch_configure(slots, capacity)                    gpu_decoder.cu:904-970
//   batch_prefill_begin(starts, lengths, slots)         the index staging of batch_prefill_embeds (:1106-1127)
//                                                       and its state publication (:1131-1150), in one copy
//   attention_block_ragged(li, q, k, v, ctx, total)     the KV body of :1025-1052 (scatter, ragged attention)
//   batch_decode_begin(slots)                           the row -> slot staging of batch_decode (:1199-1200)
//   attention_block_batch(li, q, k, v, ctx, batch)      the KV body of :972-1003 (append, batched attention)
//   batch_decode(positions, slots, io, stream)          the captured form: one graph per batch size (:1210-1213)
//   batch_slots(), batch_graph_count()                  gpu_decoder.h:85-87
//
// As in the reference, a request's whole first prefill becomes its fixed region (len = prefill = prompt
// length, ring_pos = 0) and `capacity` is the longest prompt plus the window.  New here: requests that
// name the same doc_key share the physical prefix blocks, and a slot only holds ceil(P / 16) + W / 16
// blocks instead of `capacity` rows.
// ------------------------------------------------------------------------------------------------
class UOCR_HOST_API GpuDecoderKV {
public:
    GpuDecoderKV(int num_layers, int kv_heads, int head_dim, int window, DType dtype = DType::BF16);
    ~GpuDecoderKV();
    GpuDecoderKV(const GpuDecoderKV&) = delete;
    GpuDecoderKV& operator=(const GpuDecoderKV&) = delete;

    // Returns true when device buffers were (re)allocated (captured graphs are dropped then).
    bool batch_configure(int slots, int capacity);
    int batch_slots() const;
    int batch_graph_count() const;

    // Request r owns packed rows [starts[r], starts[r] + lengths[r]) and cache slot slots[r]; doc_keys[r]
    // (optional) names a shareable prefix.  Admits the slots (one packed state upload for the wave) and
    // stages the row -> slot and row -> position arrays.  Returns the packed row count.
    int batch_prefill_begin(const std::vector<int>& starts, const std::vector<int>& lengths, const std::vector<int>& slots,
                            const std::vector<std::string>& doc_keys = {}, cudaStream_t stream = nullptr);
    void attention_block_ragged(int li, const float* q, const float* k, const float* v, float* ctx, int total, int heads,
                                cudaStream_t stream = nullptr);
    void batch_decode_begin(const std::vector<int>& slots, cudaStream_t stream = nullptr);
    void attention_block_batch(int li, const float* q, const float* k, const float* v, float* ctx, int batch, int heads,
                               cudaStream_t stream = nullptr);
    // All layers of a decode step on fixed activation buffers, replaying a graph captured on first use for
    // this batch size (io.d_slots / io.d_positions are ignored: the staged arrays of this object are used).
    // With a positive rope_theta in `io` the rotary embedding is folded into the step and `positions` are
    // staged as well; otherwise they are not needed by the KV half.
    void batch_decode(const std::vector<int>& positions, const std::vector<int>& slots, const PagedBatchKV::StepIO& io,
                      bool fold_rope, cudaStream_t stream);
    void batch_release(int slot, cudaStream_t stream = nullptr);

    PagedBatchKV& kv();
    const int* d_batch_slots() const;  // [batch] row -> slot, as staged by the last *_begin / batch_decode

private:
    struct Impl;
    std::unique_ptr<Impl> p_;
};

}  // namespace cuda
}  // namespace uocr
