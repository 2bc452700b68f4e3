// Host-side classes of the R-SWA path (see include/uocr/rswa_host.h): arena, block manager,
// scheduler, slot list, and the device-backed caches built on the C ABI.
#include "uocr/rswa_host.h"

#include <cuda_runtime.h>

#include <algorithm>
#include <cstdio>
#include <cstring>
#include <ctime>
#include <map>
#include <mutex>

namespace uocr {

namespace {

inline void cuda_ok(cudaError_t e, const char* what) {
    if (e != cudaSuccess) UOCR_THROW(std::string(what) + ": " + cudaGetErrorString(e));
}
inline void abi_ok(int rc, const char* what) {
    if (rc != UOCR_B200_OK) UOCR_THROW(std::string(what) + ": " + uocr_b200_status_string(rc) + ": " + uocr_b200_last_error());
}
inline int blocks_for(int tokens) { return (tokens + UOCR_B200_BLOCK_TOKENS - 1) / UOCR_B200_BLOCK_TOKENS; }
inline double cpu_seconds() { return static_cast<double>(::clock()) / CLOCKS_PER_SEC; }
inline bool stream_is_capturing(cudaStream_t st) {
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    return cudaStreamIsCapturing(st, &cs) == cudaSuccess && cs != cudaStreamCaptureStatusNone;
}

}  // namespace

// =================================================================================================
// MemoryPool -- behaviour of src/scheduler/memory_pool.cpp:7-85
// =================================================================================================
MemoryPool::MemoryPool(std::size_t bytes, std::size_t alignment) : alignment_(alignment) {
    if (bytes) reserve(bytes);
}

void MemoryPool::reserve(std::size_t bytes) {
    total_ = bytes;
    backing_.clear();
    reset();
}

void MemoryPool::reset() {
    used_ = peak_ = 0;
    spans_.assign(1, Block{0, total_});
}

std::uint8_t* MemoryPool::base() {
    if (backing_.size() != total_) backing_.assign(total_, 0);
    return backing_.data();
}
const std::uint8_t* MemoryPool::base() const {
    if (backing_.size() != total_) backing_.assign(total_, 0);
    return backing_.data();
}

i64 MemoryPool::allocate(std::size_t bytes, std::size_t alignment) {
    if (bytes == 0) return 0;
    std::size_t a = alignment ? alignment : alignment_;
    if (a == 0) a = 1;
    for (auto it = spans_.begin(); it != spans_.end(); ++it) {
        const std::size_t begin = it->offset, room = it->size;
        const std::size_t pad = (a - begin % a) % a;
        if (room < pad + bytes) continue;
        const std::size_t at = begin + pad;
        const std::size_t tail = room - pad - bytes;
        // the span is replaced by [pad piece][tail piece], whichever exist, keeping offset order
        if (pad && tail) {
            it->size = pad;
            spans_.insert(it + 1, Block{at + bytes, tail});
        } else if (pad) {
            it->size = pad;
        } else if (tail) {
            it->offset = at + bytes;
            it->size = tail;
        } else {
            spans_.erase(it);
        }
        used_ += pad + bytes;
        peak_ = std::max(peak_, used_);
        return static_cast<i64>(at);
    }
    return -1;
}

void MemoryPool::free(i64 offset, std::size_t bytes) {
    if (bytes == 0) return;
    const std::size_t off = static_cast<std::size_t>(offset);
    auto it = std::lower_bound(spans_.begin(), spans_.end(), off,
                               [](const Block& b, std::size_t o) { return b.offset < o; });
    it = spans_.insert(it, Block{off, bytes});
    if (used_ >= bytes) used_ -= bytes;  // alignment padding is never given back
    auto next = it + 1;
    if (next != spans_.end() && it->offset + it->size == next->offset) {
        it->size += next->size;
        it = spans_.erase(next) - 1;
    }
    if (it != spans_.begin()) {
        auto prev = it - 1;
        if (prev->offset + prev->size == it->offset) {
            prev->size += it->size;
            spans_.erase(it);
        }
    }
}

double MemoryPool::fragmentation() const {
    std::size_t all = 0, biggest = 0;
    for (const Block& b : spans_) {
        all += b.size;
        biggest = std::max(biggest, b.size);
    }
    return all ? 1.0 - static_cast<double>(biggest) / static_cast<double>(all) : 0.0;
}

// =================================================================================================
// BlockManager -- behaviour of src/scheduler/block_manager.cpp:7-77
// =================================================================================================
BlockManager::BlockManager(std::size_t prefix_pool_bytes, std::size_t ring_pool_bytes)
    : prefix_arena_(prefix_pool_bytes), ring_arena_(ring_pool_bytes) {}

void BlockManager::refresh_shared() {
    std::size_t s = 0;
    for (const auto& kv : table_)
        if (kv.second.refcount >= 2) s += kv.second.bytes;
    shared_now_ = s;
    shared_peak_ = std::max(shared_peak_, s);
}

PrefixEntry* BlockManager::acquire_prefix(const std::string& key, int prefill_len, std::size_t bytes) {
    auto hit = table_.find(key);
    if (hit == table_.end()) {
        const i64 off = prefix_arena_.allocate(bytes);
        UOCR_CHECK(off >= 0, "prefix pool exhausted");
        PrefixEntry fresh;
        fresh.key = key;
        fresh.prefill_len = prefill_len;
        fresh.bytes = bytes;
        fresh.refcount = 0;
        fresh.offset = off;
        hit = table_.emplace(key, std::move(fresh)).first;
    }
    hit->second.refcount += 1;
    refresh_shared();
    return &hit->second;
}

void BlockManager::release_prefix(const std::string& key) {
    auto hit = table_.find(key);
    if (hit == table_.end()) return;  // unknown key: nothing to do
    if (--hit->second.refcount <= 0) {
        prefix_arena_.free(hit->second.offset, hit->second.bytes);
        table_.erase(hit);
    }
    refresh_shared();
}

i64 BlockManager::allocate_ring(std::size_t bytes) { return ring_arena_.allocate(bytes); }
void BlockManager::free_ring(i64 offset, std::size_t bytes) { ring_arena_.free(offset, bytes); }

std::size_t BlockManager::total_prefix_bytes() const {
    std::size_t t = 0;
    for (const auto& kv : table_) t += kv.second.bytes;
    return t;
}

BlockManager::Stats BlockManager::stats() const {
    Stats s;
    s.prefix_live_bytes = prefix_arena_.used();
    s.prefix_peak_bytes = prefix_arena_.peak();
    s.prefix_shared_bytes = shared_now_;
    s.ring_live_bytes = ring_arena_.used();
    s.ring_peak_bytes = ring_arena_.peak();
    s.prefix_fragmentation = prefix_arena_.fragmentation();
    s.ring_fragmentation = ring_arena_.fragmentation();
    s.live_prefixes = table_.size();
    return s;
}

// =================================================================================================
// ContinuousBatchScheduler -- behaviour of src/scheduler/continuous_batch.cpp:10-117
// =================================================================================================
int ContinuousBatchScheduler::add_request(Request r) {
    const int id = next_id_++;
    r.id = id;
    if (r.arrival_time == 0.0) r.arrival_time = cpu_seconds();
    queue_.push_back(id);
    all_.emplace(id, std::move(r));
    return id;
}

Batch ContinuousBatchScheduler::build_batch() {
    Batch out;
    auto filled = [&] { return static_cast<int>(out.prefill.size() + out.decode.size()); };
    // requests already running keep their place first
    for (int id : active_) {
        auto it = all_.find(id);
        if (it == all_.end() || it->second.is_finished()) continue;
        if (filled() >= max_batch_) break;
        if (it->second.state == ReqState::Decoding) out.decode.push_back(id);
        else if (it->second.state == ReqState::Prefilling) out.prefill.push_back(id);
    }
    // then admit from the FIFO while there is room
    while (!queue_.empty() && filled() < max_batch_) {
        const int id = queue_.front();
        queue_.pop_front();
        auto it = all_.find(id);
        if (it == all_.end()) continue;
        it->second.state = ReqState::Prefilling;
        active_.push_back(id);
        out.prefill.push_back(id);
    }
    // drop what has finished in the meantime
    std::vector<int> keep;
    keep.reserve(active_.size());
    for (int id : active_) {
        auto it = all_.find(id);
        if (it != all_.end() && !it->second.is_finished()) keep.push_back(id);
    }
    active_.swap(keep);
    return out;
}

void ContinuousBatchScheduler::mark_prefilling(int id) {
    if (Request* r = get(id)) r->state = ReqState::Prefilling;
}

void ContinuousBatchScheduler::mark_prefilled(int id) {
    if (Request* r = get(id)) {
        r->state = ReqState::Decoding;
        r->prefill_time = cpu_seconds();
    }
}

bool ContinuousBatchScheduler::add_token(int id, int token) {
    Request* r = get(id);
    if (!r) return true;
    r->output_tokens.push_back(token);
    r->decode_steps += 1;
    if (r->first_token_time == 0.0) r->first_token_time = cpu_seconds();
    if (static_cast<int>(r->output_tokens.size()) < r->max_new_tokens) return false;
    finish(id);
    return true;
}

void ContinuousBatchScheduler::finish(int id) {
    Request* r = get(id);
    if (!r) return;
    r->state = ReqState::Finished;
    r->finish_time = cpu_seconds();
    r->cache.reset();
    active_.erase(std::remove(active_.begin(), active_.end(), id), active_.end());
}

Request* ContinuousBatchScheduler::get(int id) {
    auto it = all_.find(id);
    return it == all_.end() ? nullptr : &it->second;
}
const Request* ContinuousBatchScheduler::get(int id) const {
    auto it = all_.find(id);
    return it == all_.end() ? nullptr : &it->second;
}

ContinuousBatchScheduler::Stats ContinuousBatchScheduler::stats() const {
    Stats s;
    s.total_requests = all_.size();
    for (const auto& kv : all_) {
        if (!kv.second.is_finished()) continue;
        s.finished_requests += 1;
        s.prefill_tokens += kv.second.prompt_tokens.size();
        s.decode_tokens += kv.second.output_tokens.size();
    }
    s.waiting = queue_.size();
    s.running = active_.size();
    s.last_batch_size = static_cast<double>(active_.size());
    return s;
}

// =================================================================================================
// SlotAllocator -- src/engine/engine.cpp:306-318, 341-347
// =================================================================================================
void SlotAllocator::reset(int slots) {
    free_.resize(static_cast<std::size_t>(std::max(slots, 0)));
    for (int i = 0; i < slots; ++i) free_[static_cast<std::size_t>(i)] = i;
    by_request_.clear();
}

int SlotAllocator::acquire(int request_id) {
    UOCR_CHECK(!free_.empty(), "generate_batch: no free slot");
    const int slot = free_.back();
    free_.pop_back();
    by_request_[request_id] = slot;
    return slot;
}

void SlotAllocator::release(int request_id) {
    auto it = by_request_.find(request_id);
    if (it == by_request_.end()) return;
    free_.push_back(it->second);
    by_request_.erase(it);
}

int SlotAllocator::slot_of(int request_id) const {
    auto it = by_request_.find(request_id);
    return it == by_request_.end() ? -1 : it->second;
}

// =================================================================================================
// detail::PagedSeqStore -- one sequence, all layers, private blocks, device cursors + host shadow
// =================================================================================================
namespace detail {

class PagedSeqStore {
public:
    int layers = 0, kvh = 0, hd = 0, window = 128;
    int prefill_len = 0, capacity = 0;
    bool configured = false;
    DType dtype = DType::F32;

    // host shadow of the state machine (the device cursors advance identically)
    std::vector<int> len, ring_pos;
    std::vector<char> ring_started;

    // device side
    int n_blocks = 0, alloc_rows = 0;
    std::vector<void*> kpool, vpool;  // per layer
    int32_t* d_table = nullptr;
    int* d_len = nullptr;       // [layers]
    int* d_ring = nullptr;      // [layers]
    int* d_prefill = nullptr;   // [1]
    int* d_zero_slots = nullptr;  // [alloc_rows] zeros (row -> slot 0)
    int* d_iota = nullptr;        // [alloc_rows] 0,1,2,...
    float* d_stage_a = nullptr;   // staging for k / q / gathered K
    float* d_stage_b = nullptr;   // staging for v / out / gathered V
    std::size_t stage_elems = 0;
    uocr_b200_workspace* ws = nullptr;
    std::vector<uocr_b200_paged_kv> view;

    // host mirrors (logical view, [capacity][row])
    mutable std::vector<std::vector<float>> kmir, vmir;
    mutable std::vector<char> mirror_fresh;  // mirror equals device
    std::vector<char> host_dirty;            // caller may have written through mutable_*()

    ~PagedSeqStore() { release_device(); }

    int row() const { return kvh * hd; }
    int esize() const { return dtype == DType::BF16 ? 2 : 4; }

    void release_device() {
        for (void* p : kpool) if (p) cudaFree(p);
        for (void* p : vpool) if (p) cudaFree(p);
        kpool.clear();
        vpool.clear();
        for (void* p : {static_cast<void*>(d_table), static_cast<void*>(d_len), static_cast<void*>(d_ring),
                        static_cast<void*>(d_prefill), static_cast<void*>(d_zero_slots), static_cast<void*>(d_iota),
                        static_cast<void*>(d_stage_a), static_cast<void*>(d_stage_b)})
            if (p) cudaFree(p);
        d_table = nullptr; d_len = d_ring = d_prefill = d_zero_slots = d_iota = nullptr;
        d_stage_a = d_stage_b = nullptr;
        stage_elems = 0;
        if (ws) uocr_b200_workspace_destroy(ws);
        ws = nullptr;
        n_blocks = alloc_rows = 0;
    }

    void configure(int L, int kv_heads, int head_dim, int W) {
        release_device();
        layers = L; kvh = kv_heads; hd = head_dim; window = W;
        len.assign(static_cast<std::size_t>(L), 0);
        ring_pos.assign(static_cast<std::size_t>(L), 0);
        ring_started.assign(static_cast<std::size_t>(L), 0);
        kmir.assign(static_cast<std::size_t>(L), {});
        vmir.assign(static_cast<std::size_t>(L), {});
        mirror_fresh.assign(static_cast<std::size_t>(L), 0);
        host_dirty.assign(static_cast<std::size_t>(L), 0);
        prefill_len = capacity = 0;
        configured = true;
    }

    void ensure_stage(std::size_t elems) {
        if (elems <= stage_elems) return;
        if (d_stage_a) cudaFree(d_stage_a);
        if (d_stage_b) cudaFree(d_stage_b);
        cuda_ok(cudaMalloc(&d_stage_a, elems * sizeof(float)), "stage alloc");
        cuda_ok(cudaMalloc(&d_stage_b, elems * sizeof(float)), "stage alloc");
        stage_elems = elems;
    }

    void publish_cursors(cudaStream_t st = nullptr) {
        cuda_ok(cudaMemcpyAsync(d_len, len.data(), sizeof(int) * layers, cudaMemcpyHostToDevice, st), "len H2D");
        cuda_ok(cudaMemcpyAsync(d_ring, ring_pos.data(), sizeof(int) * layers, cudaMemcpyHostToDevice, st), "ring H2D");
        cuda_ok(cudaMemcpyAsync(d_prefill, &prefill_len, sizeof(int), cudaMemcpyHostToDevice, st), "prefill H2D");
        cuda_ok(cudaStreamSynchronize(st), "cursor publish");  // sources are host members
    }

    void reset(int P) {
        UOCR_CHECK(configured, "RSWACache not configured");
        UOCR_CHECK(P >= 0, "prefill_len must be >= 0");
        UOCR_CHECK(layers > 0 && kvh > 0 && hd > 0 && window > 0, "RSWACache geometry must be positive");
        prefill_len = P;
        capacity = P + window;
        const int need_blocks = blocks_for(P) + blocks_for(window) + 1;
        const int need_rows = need_blocks * UOCR_B200_BLOCK_TOKENS;
        const std::size_t blk_bytes = static_cast<std::size_t>(kvh) * UOCR_B200_BLOCK_TOKENS * hd * esize();
        if (need_blocks > n_blocks || kpool.empty()) {
            release_device();
            kpool.assign(static_cast<std::size_t>(layers), nullptr);
            vpool.assign(static_cast<std::size_t>(layers), nullptr);
            for (int l = 0; l < layers; ++l) {
                cuda_ok(cudaMalloc(&kpool[l], blk_bytes * need_blocks), "K pool");
                cuda_ok(cudaMalloc(&vpool[l], blk_bytes * need_blocks), "V pool");
            }
            n_blocks = need_blocks;
            alloc_rows = need_rows;
            cuda_ok(cudaMalloc(&d_table, sizeof(int32_t) * need_blocks), "table");
            cuda_ok(cudaMalloc(&d_len, sizeof(int) * layers), "len");
            cuda_ok(cudaMalloc(&d_ring, sizeof(int) * layers), "ring");
            cuda_ok(cudaMalloc(&d_prefill, sizeof(int)), "prefill");
            cuda_ok(cudaMalloc(&d_zero_slots, sizeof(int) * need_rows), "slots");
            cuda_ok(cudaMalloc(&d_iota, sizeof(int) * need_rows), "iota");
            std::vector<int> iota(static_cast<std::size_t>(need_rows));
            for (int i = 0; i < need_rows; ++i) iota[static_cast<std::size_t>(i)] = i;
            cuda_ok(cudaMemcpy(d_iota, iota.data(), sizeof(int) * need_rows, cudaMemcpyHostToDevice), "iota H2D");
            cuda_ok(cudaMemset(d_zero_slots, 0, sizeof(int) * need_rows), "slots zero");
            std::vector<int32_t> tbl(static_cast<std::size_t>(need_blocks));
            for (int i = 0; i < need_blocks; ++i) tbl[static_cast<std::size_t>(i)] = i;
            cuda_ok(cudaMemcpy(d_table, tbl.data(), sizeof(int32_t) * need_blocks, cudaMemcpyHostToDevice), "table H2D");
            abi_ok(uocr_b200_workspace_create(std::max(need_rows, 64), &ws), "workspace");
            view.assign(static_cast<std::size_t>(layers), uocr_b200_paged_kv{});
            for (int l = 0; l < layers; ++l) {
                view[l].k_pool = kpool[l];
                view[l].v_pool = vpool[l];
                view[l].block_table = d_table;
                view[l].table_stride = need_blocks;
                view[l].num_blocks = need_blocks;
                view[l].kv_heads = kvh;
                view[l].head_dim = hd;
                view[l].dtype = dtype == DType::BF16 ? UOCR_B200_BF16 : UOCR_B200_F32;
            }
        }
        for (int l = 0; l < layers; ++l) {
            cuda_ok(cudaMemset(kpool[l], 0, blk_bytes * n_blocks), "K zero");
            cuda_ok(cudaMemset(vpool[l], 0, blk_bytes * n_blocks), "V zero");
            len[l] = P;
            ring_pos[l] = 0;
            ring_started[l] = 0;
            kmir[l].assign(static_cast<std::size_t>(capacity) * row(), 0.0f);
            vmir[l].assign(static_cast<std::size_t>(capacity) * row(), 0.0f);
            mirror_fresh[l] = 1;  // all zeros on both sides
            host_dirty[l] = 0;
        }
        publish_cursors();
    }

    // Physical "position" (token index along the table row) of logical slot s.
    int phys_pos(int s) const {
        return s < prefill_len ? s : blocks_for(prefill_len) * UOCR_B200_BLOCK_TOKENS + (s - prefill_len);
    }

    // If the caller wrote through mutable_keys()/mutable_values(), push the mirror back first.
    void flush_host_edits(int layer) {
        if (!host_dirty[layer]) return;
        const int n = len[layer];
        if (n > 0) {
            ensure_stage(static_cast<std::size_t>(capacity) * row());
            std::vector<int> pos(static_cast<std::size_t>(n));
            for (int s = 0; s < n; ++s) pos[static_cast<std::size_t>(s)] = phys_pos(s);
            int* d_pos = nullptr;
            cuda_ok(cudaMalloc(&d_pos, sizeof(int) * n), "pos alloc");
            cuda_ok(cudaMemcpy(d_pos, pos.data(), sizeof(int) * n, cudaMemcpyHostToDevice), "pos H2D");
            cuda_ok(cudaMemcpy(d_stage_a, kmir[layer].data(), sizeof(float) * n * row(), cudaMemcpyHostToDevice), "K H2D");
            cuda_ok(cudaMemcpy(d_stage_b, vmir[layer].data(), sizeof(float) * n * row(), cudaMemcpyHostToDevice), "V H2D");
            abi_ok(uocr_b200_rswa_write_prefill_ragged_paged(&view[layer], d_stage_a, d_stage_b, d_zero_slots, d_pos, n,
                                                             ws, nullptr), "mirror upload");
            cuda_ok(cudaDeviceSynchronize(), "mirror upload sync");
            cudaFree(d_pos);
        }
        host_dirty[layer] = 0;
        mirror_fresh[layer] = 0;  // a bf16 pool rounds what was written
    }

    void advance_shadow(int layer) {
        const int n = len[layer];
        if (n < prefill_len + window) {
            len[layer] = n + 1;
            if (n + 1 >= prefill_len + window) {
                ring_started[layer] = 1;
                ring_pos[layer] = 0;
            }
        } else {
            ring_started[layer] = 1;
            ring_pos[layer] = (ring_pos[layer] + 1) % window;
        }
    }

    void write_prefill_dev(int layer, const float* d_k, const float* d_v, int seq, cudaStream_t st) {
        UOCR_CHECK(seq <= capacity, "prefill larger than cache capacity");
        flush_host_edits(layer);
        if (seq > 0)
            abi_ok(uocr_b200_rswa_write_prefill_ragged_paged(&view[layer], d_k, d_v, d_zero_slots, d_iota, seq, ws, st),
                   "write_prefill");
        len[layer] = seq;
        prefill_len = seq;
        cuda_ok(cudaMemcpyAsync(d_len + layer, &len[layer], sizeof(int), cudaMemcpyHostToDevice, st), "len H2D");
        cuda_ok(cudaMemcpyAsync(d_prefill, &prefill_len, sizeof(int), cudaMemcpyHostToDevice, st), "prefill H2D");
        cuda_ok(cudaStreamSynchronize(st), "write_prefill sync");
        mirror_fresh[layer] = 0;
    }

    void append_dev(int layer, const float* d_k, const float* d_v, cudaStream_t st) {
        flush_host_edits(layer);
        abi_ok(uocr_b200_rswa_append_decode_batch_paged(&view[layer], d_k, d_v, d_len + layer, d_ring + layer, d_prefill,
                                                        d_zero_slots, 1, window, ws, st), "append_decode");
        advance_shadow(layer);
        mirror_fresh[layer] = 0;
    }

    void attention_dev(int layer, const float* d_q, int seq, int q_start, float* d_out, int heads, bool causal,
                       cudaStream_t st) {
        flush_host_edits(layer);
        if (seq > ws_rows()) grow_workspace(seq);
        abi_ok(uocr_b200_rswa_attention_paged(&view[layer], 0, d_q, len[layer], nullptr, prefill_len, nullptr, seq,
                                              q_start, heads, causal ? 1 : 0, d_out, ws, st), "attention");
    }

    // The same attention over the DEVICE cursors: nothing of the host shadow is frozen into the launch.
    void attention_devlen_dev(int layer, const float* d_q, int seq, int q_start, float* d_out, int heads, bool causal,
                              cudaStream_t st) {
        UOCR_CHECK(!host_dirty[layer], "attention_devlen: pending host edits (mutable_keys/values) must be flushed outside capture");
        UOCR_CHECK(seq <= ws_rows(), "attention_devlen: more query rows than the cache's workspace holds");
        abi_ok(uocr_b200_rswa_attention_paged(&view[layer], 0, d_q, 0, d_len + layer, 0, d_prefill, seq, q_start, heads,
                                              causal ? 1 : 0, d_out, ws, st), "attention_devlen");
    }

    int ws_rows_ = 0;
    int ws_rows() { return ws_rows_ ? ws_rows_ : std::max(alloc_rows, 64); }
    void grow_workspace(int rows) {
        cuda_ok(cudaDeviceSynchronize(), "workspace grow sync");
        if (ws) uocr_b200_workspace_destroy(ws);
        ws = nullptr;
        abi_ok(uocr_b200_workspace_create(rows, &ws), "workspace");
        ws_rows_ = rows;
    }

    // Fills the device staging buffers with the logical fp32 view of `layer` (rows >= len are zero).
    void gather_dev(int layer, cudaStream_t st) {
        flush_host_edits(layer);
        ensure_stage(static_cast<std::size_t>(std::max(capacity, 1)) * row());
        if (capacity > 0)
            abi_ok(uocr_b200_rswa_gather_paged(&view[layer], d_len + layer, d_prefill, d_zero_slots, 1, capacity, d_stage_a,
                                               d_stage_b, UOCR_B200_F32, ws, st), "gather");
    }

    void refresh_mirror(int layer) const {
        auto* self = const_cast<PagedSeqStore*>(this);
        if (mirror_fresh[layer] || capacity == 0) return;
        self->gather_dev(layer, nullptr);
        const std::size_t n = static_cast<std::size_t>(capacity) * row();
        kmir[layer].resize(n);
        vmir[layer].resize(n);
        cuda_ok(cudaMemcpy(kmir[layer].data(), d_stage_a, n * sizeof(float), cudaMemcpyDeviceToHost), "K D2H");
        cuda_ok(cudaMemcpy(vmir[layer].data(), d_stage_b, n * sizeof(float), cudaMemcpyDeviceToHost), "V D2H");
        mirror_fresh[layer] = 1;
    }
};

}  // namespace detail

// =================================================================================================
// RSWACache -- interface of include/uocr/kv_cache.h:23-86, semantics of src/scheduler/kv_cache.cpp
// =================================================================================================
RSWACache::RSWACache() : s_(new detail::PagedSeqStore) {}
RSWACache::RSWACache(int num_layers, int kv_heads, int head_dim, int window) : s_(new detail::PagedSeqStore) {
    configure(num_layers, kv_heads, head_dim, window);
}
RSWACache::~RSWACache() = default;
RSWACache::RSWACache(RSWACache&&) noexcept = default;
RSWACache& RSWACache::operator=(RSWACache&&) noexcept = default;

void RSWACache::configure(int num_layers, int kv_heads, int head_dim, int window) {
    s_->configure(num_layers, kv_heads, head_dim, window);
}
void RSWACache::set_kv_dtype(DType t) {
    UOCR_CHECK(t == DType::F32 || t == DType::BF16, "KV dtype must be F32 or BF16");
    UOCR_CHECK(s_->kpool.empty(), "set_kv_dtype must precede reset()");
    s_->dtype = t;
}
void RSWACache::reset(int prefill_len) { s_->reset(prefill_len); }

int RSWACache::num_layers() const { return s_->layers; }
int RSWACache::kv_heads() const { return s_->kvh; }
int RSWACache::head_dim() const { return s_->hd; }
int RSWACache::window() const { return s_->window; }
int RSWACache::prefill_len() const { return s_->prefill_len; }
int RSWACache::length(int layer) const { return s_->len[layer]; }
int RSWACache::ring_pos(int layer) const { return s_->ring_pos[layer]; }
bool RSWACache::ring_started(int layer) const { return s_->ring_started[layer] != 0; }
int RSWACache::capacity() const { return s_->capacity; }

void RSWACache::write_prefill(int layer, const float* k, const float* v, int seq) {
    UOCR_CHECK(seq <= s_->capacity, "prefill larger than cache capacity");
    s_->flush_host_edits(layer);  // before the staging buffers are reused for k / v
    const std::size_t n = static_cast<std::size_t>(std::max(seq, 0)) * s_->row();
    s_->ensure_stage(std::max<std::size_t>(n, 1));
    if (n) {
        cuda_ok(cudaMemcpy(s_->d_stage_a, k, n * sizeof(float), cudaMemcpyHostToDevice), "K H2D");
        cuda_ok(cudaMemcpy(s_->d_stage_b, v, n * sizeof(float), cudaMemcpyHostToDevice), "V H2D");
    }
    s_->write_prefill_dev(layer, s_->d_stage_a, s_->d_stage_b, seq, nullptr);
}

void RSWACache::append_decode(int layer, const float* k, const float* v) {
    s_->flush_host_edits(layer);
    const std::size_t n = static_cast<std::size_t>(s_->row());
    s_->ensure_stage(n);
    cuda_ok(cudaMemcpy(s_->d_stage_a, k, n * sizeof(float), cudaMemcpyHostToDevice), "K H2D");
    cuda_ok(cudaMemcpy(s_->d_stage_b, v, n * sizeof(float), cudaMemcpyHostToDevice), "V H2D");
    s_->append_dev(layer, s_->d_stage_a, s_->d_stage_b, nullptr);
}

void RSWACache::attention(int layer, const float* q, int seq, int q_start, float* out, int heads, bool causal) const {
    UOCR_CHECK(s_->hd <= 512, "head_dim too large for stack accumulator");
    if (seq <= 0) return;
    s_->flush_host_edits(layer);
    const std::size_t n = static_cast<std::size_t>(seq) * heads * s_->hd;
    s_->ensure_stage(n);
    cuda_ok(cudaMemcpy(s_->d_stage_a, q, n * sizeof(float), cudaMemcpyHostToDevice), "q H2D");
    s_->attention_dev(layer, s_->d_stage_a, seq, q_start, s_->d_stage_b, heads, causal, nullptr);
    cuda_ok(cudaMemcpy(out, s_->d_stage_b, n * sizeof(float), cudaMemcpyDeviceToHost), "out D2H");
}

const float* RSWACache::keys(int layer) const {
    s_->refresh_mirror(layer);
    return s_->kmir[layer].data();
}
const float* RSWACache::values(int layer) const {
    s_->refresh_mirror(layer);
    return s_->vmir[layer].data();
}
float* RSWACache::mutable_keys(int layer) {
    s_->refresh_mirror(layer);
    s_->host_dirty[layer] = 1;
    return s_->kmir[layer].data();
}
float* RSWACache::mutable_values(int layer) {
    s_->refresh_mirror(layer);
    s_->host_dirty[layer] = 1;
    return s_->vmir[layer].data();
}

std::size_t RSWACache::bytes() const {
    // the reference reports its fp32 footprint: 2 x layers x capacity x row x 4 (kv_cache.cpp:132-137)
    return 2u * static_cast<std::size_t>(s_->layers) * s_->capacity * s_->row() * sizeof(float);
}

// =================================================================================================
// cuda::GpuRSWACache -- interface of include/uocr/gpu_cache.h:21-72
// =================================================================================================
namespace cuda {

GpuRSWACache::GpuRSWACache() : s_(new detail::PagedSeqStore) {}
GpuRSWACache::GpuRSWACache(int num_layers, int kv_heads, int head_dim, int window) : s_(new detail::PagedSeqStore) {
    configure(num_layers, kv_heads, head_dim, window);
}
GpuRSWACache::~GpuRSWACache() = default;

void GpuRSWACache::configure(int num_layers, int kv_heads, int head_dim, int window) {
    s_->configure(num_layers, kv_heads, head_dim, window);
}
void GpuRSWACache::set_kv_dtype(DType t) {
    UOCR_CHECK(t == DType::F32 || t == DType::BF16, "KV dtype must be F32 or BF16");
    UOCR_CHECK(s_->kpool.empty(), "set_kv_dtype must precede reset()");
    s_->dtype = t;
}
void GpuRSWACache::reset(int prefill_len) {
    UOCR_CHECK(s_->configured, "GpuRSWACache not configured");
    s_->reset(prefill_len);
}
void GpuRSWACache::write_prefill(int layer, const float* d_k, const float* d_v, int seq, cudaStream_t stream) {
    s_->write_prefill_dev(layer, d_k, d_v, seq, stream);
}
void GpuRSWACache::append_decode(int layer, const float* d_k, const float* d_v, cudaStream_t stream) {
    s_->append_dev(layer, d_k, d_v, stream);
}
void GpuRSWACache::reset_device_state(int prefill_len, cudaStream_t stream) {
    // device cursors <- (len = prefill_len, ring_pos = 0) for every layer (src/kernels/cuda/gpu_cache.cu:88-95)
    for (int l = 0; l < s_->layers; ++l) {
        s_->len[l] = prefill_len;
        s_->ring_pos[l] = 0;
        s_->ring_started[l] = 0;
    }
    s_->prefill_len = prefill_len;
    s_->publish_cursors(stream);
}
void GpuRSWACache::append_decode_device(int layer, const float* d_k, const float* d_v, cudaStream_t stream) {
    s_->append_dev(layer, d_k, d_v, stream);
}
const int* GpuRSWACache::len_dev(int layer) const { return s_->d_len + layer; }
void GpuRSWACache::attention(int layer, const float* d_q, int seq, int q_start, float* d_out, int heads, bool causal,
                             cudaStream_t stream) const {
    s_->attention_dev(layer, d_q, seq, q_start, d_out, heads, causal, stream);
}
void GpuRSWACache::attention_devlen(int layer, const float* d_q, int seq, int q_start, float* d_out, int heads,
                                    bool causal, cudaStream_t stream) const {
    s_->attention_devlen_dev(layer, d_q, seq, q_start, d_out, heads, causal, stream);
}
int GpuRSWACache::len(int layer) const { return s_->len[layer]; }
int GpuRSWACache::prefill_len() const { return s_->prefill_len; }
int GpuRSWACache::window() const { return s_->window; }
int GpuRSWACache::capacity() const { return s_->capacity; }
int GpuRSWACache::num_layers() const { return s_->layers; }
const float* GpuRSWACache::keys(int layer, cudaStream_t stream) const {
    UOCR_CHECK(!stream_is_capturing(stream), "GpuRSWACache::keys: a snapshot cannot be taken inside stream capture; use attention_devlen");
    s_->gather_dev(layer, stream);
    return s_->d_stage_a;
}
const float* GpuRSWACache::values(int layer, cudaStream_t stream) const {
    UOCR_CHECK(!stream_is_capturing(stream), "GpuRSWACache::values: a snapshot cannot be taken inside stream capture; use attention_devlen");
    s_->gather_dev(layer, stream);
    return s_->d_stage_b;
}

// =================================================================================================
// the reference's free functions (include/uocr/cuda_ops.h:59-123) over the C ABI
// =================================================================================================
namespace {

// One workspace per (device, stream), never freed or moved once a launch may have used it.
struct StreamScratch {
    uocr_b200_workspace* ws = nullptr;
    int rows = 0;
};
std::mutex g_scratch_mutex;
std::map<std::pair<int, cudaStream_t>, StreamScratch> g_scratch;
std::vector<uocr_b200_workspace*> g_retired;  // superseded by a larger one; kept alive for captured graphs

constexpr int kDefaultScratchRows = 4096;

bool prepare_scratch(cudaStream_t stream, int rows) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return false;
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    StreamScratch& s = g_scratch[{dev, stream}];
    if (s.ws && rows <= s.rows) return true;
    if (stream_is_capturing(stream)) {
        std::fprintf(stderr, "uocr::cuda: no scratch for %d rows on this stream and the stream is capturing: call "
                             "rswa_prepare(stream, max_rows) before the capture begins\n", rows);
        return false;
    }
    uocr_b200_workspace* fresh = nullptr;
    if (uocr_b200_workspace_create(rows, &fresh) != UOCR_B200_OK) {
        std::fprintf(stderr, "uocr::cuda: workspace: %s\n", uocr_b200_last_error());
        return false;
    }
    if (s.ws) g_retired.push_back(s.ws);
    s.ws = fresh;
    s.rows = rows;
    return true;
}

// The workspace of `stream` for a call with `rows` query rows; null (nothing may be launched) when the
// prepared one is too small or none exists and none can be made now.
uocr_b200_workspace* default_workspace(cudaStream_t stream, int rows) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
    {
        std::lock_guard<std::mutex> lock(g_scratch_mutex);
        auto it = g_scratch.find({dev, stream});
        if (it != g_scratch.end() && it->second.ws) {
            if (rows <= it->second.rows) return it->second.ws;
            std::fprintf(stderr, "uocr::cuda: %d query rows exceed the %d this stream's scratch was prepared for: call "
                                 "rswa_prepare(stream, max_rows) first (outside stream capture)\n", rows, it->second.rows);
            return nullptr;
        }
    }
    if (!prepare_scratch(stream, std::max(rows, kDefaultScratchRows))) return nullptr;
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    return g_scratch[{dev, stream}].ws;
}

// CUDA-side failures are reported, not thrown, like the reference's wrappers (gpu_cache.cu:10-18).
void report(int rc, const char* what) {
    if (rc != UOCR_B200_OK) std::fprintf(stderr, "uocr::cuda::%s: %s: %s\n", what, uocr_b200_status_string(rc), uocr_b200_last_error());
}

}  // namespace

bool rswa_prepare(cudaStream_t stream, int max_rows) { return max_rows > 0 && prepare_scratch(stream, max_rows); }

void rswa_attention_decode(const float* q, const float* kcache, const float* vcache, int kv_len, int heads,
                           int kv_heads, int head_dim, float* out, cudaStream_t stream) {
    uocr_b200_workspace* ws = default_workspace(stream, 1);
    if (!ws) return;
    report(uocr_b200_rswa_attention_f32(q, kcache, vcache, kv_len, nullptr, 1, 0, heads, kv_heads, head_dim, 0, out,
                                        ws, stream), "rswa_attention_decode");
}
void rswa_attention(const float* q, const float* kcache, const float* vcache, int kv_len, int seq, int q_start,
                    int heads, int kv_heads, int head_dim, bool causal, float* out, cudaStream_t stream) {
    if (seq <= 0) return;
    uocr_b200_workspace* ws = default_workspace(stream, seq);
    if (!ws) return;
    report(uocr_b200_rswa_attention_f32(q, kcache, vcache, kv_len, nullptr, seq, q_start, heads, kv_heads, head_dim,
                                        causal ? 1 : 0, out, ws, stream), "rswa_attention");
}
void rswa_attention_devlen(const float* q, const float* kcache, const float* vcache, const int* d_len, int seq,
                           int q_start, int heads, int kv_heads, int head_dim, bool causal, float* out,
                           cudaStream_t stream) {
    if (seq <= 0) return;
    uocr_b200_workspace* ws = default_workspace(stream, seq);
    if (!ws) return;
    report(uocr_b200_rswa_attention_f32(q, kcache, vcache, 0, d_len, seq, q_start, heads, kv_heads, head_dim,
                                        causal ? 1 : 0, out, ws, stream), "rswa_attention_devlen");
}
void rswa_append_decode(const float* k, const float* v, float* kcache, float* vcache, int* d_len, int* d_ring_pos,
                        int prefill_len, int window, int kv_heads, int head_dim, cudaStream_t stream) {
    report(uocr_b200_rswa_append_decode_f32(k, v, kcache, vcache, d_len, d_ring_pos, prefill_len, window, kv_heads,
                                            head_dim, stream), "rswa_append_decode");
}
void rswa_append_decode_batch(const float* k, const float* v, float* kcache_base, float* vcache_base, int* d_len,
                              int* d_ring_pos, const int* d_prefill_len, const int* d_slots, int batch, int batch_cap,
                              int window, int kv_heads, int head_dim, cudaStream_t stream) {
    report(uocr_b200_rswa_append_decode_batch_f32(k, v, kcache_base, vcache_base, d_len, d_ring_pos, d_prefill_len,
                                                  d_slots, batch, batch_cap, window, kv_heads, head_dim, stream),
           "rswa_append_decode_batch");
}
void rswa_attention_batch(const float* q, const float* kcache_base, const float* vcache_base, const int* d_len,
                          const int* d_slots, int batch, int batch_cap, int heads, int kv_heads, int head_dim,
                          float* out, cudaStream_t stream) {
    if (batch <= 0) return;
    uocr_b200_workspace* ws = default_workspace(stream, batch);
    if (!ws) return;
    report(uocr_b200_rswa_attention_batch_f32(q, kcache_base, vcache_base, d_len, d_slots, batch, batch_cap, heads,
                                              kv_heads, head_dim, out, ws, stream),
           "rswa_attention_batch");
}
void rswa_write_prefill_ragged(const float* k, const float* v, float* kcache_base, float* vcache_base,
                               const int* d_slots, const int* d_pos, int total, int batch_cap, int kv_heads,
                               int head_dim, cudaStream_t stream) {
    report(uocr_b200_rswa_write_prefill_ragged_f32(k, v, kcache_base, vcache_base, d_slots, d_pos, total, batch_cap,
                                                   kv_heads, head_dim, stream), "rswa_write_prefill_ragged");
}
void rswa_attention_ragged(const float* q, const float* kcache_base, const float* vcache_base, const int* d_slots,
                           const int* d_pos, int total, int batch_cap, int heads, int kv_heads, int head_dim,
                           float* out, cudaStream_t stream) {
    if (total <= 0) return;
    uocr_b200_workspace* ws = default_workspace(stream, total);
    if (!ws) return;
    report(uocr_b200_rswa_attention_ragged_f32(q, kcache_base, vcache_base, d_slots, d_pos, total, batch_cap, heads,
                                               kv_heads, head_dim, out, ws, stream),
           "rswa_attention_ragged");
}

// =================================================================================================
// PagedBatchKV
// =================================================================================================
struct PagedBatchKV::Impl {
    Config cfg;
    std::unique_ptr<BlockManager> bm;
    int stride = 0, num_blocks = 0;
    std::vector<void*> kpool, vpool;
    int32_t* d_table = nullptr;
    int* d_len = nullptr;      // [layers][slots]
    int* d_ring = nullptr;     // [layers][slots]
    int* d_prefill = nullptr;  // [slots]
    // packed slot-state records ([slot, length, write_row, row[stride]] each): two pinned staging buffers
    // used alternately, each with its device twin and an event recorded behind the copy that reads it
    int* h_stage[2] = {nullptr, nullptr};
    int* d_stage[2] = {nullptr, nullptr};
    cudaEvent_t stage_done[2] = {nullptr, nullptr};
    bool stage_used[2] = {false, false};
    int stage_next = 0;
    // captured decode steps, one per batch size
    struct StepGraph {
        cudaGraph_t graph = nullptr;
        cudaGraphExec_t exec = nullptr;
        StepIO io;
    };
    std::map<int, StepGraph> step_graphs;
    uocr_b200_workspace* ws = nullptr;
    std::vector<uocr_b200_paged_kv> view;
    struct SlotState {
        bool bound = false;
        std::string key;
        bool has_prefix = false;
        i64 ring_off = -1;
        int prefix_len = 0;
    };
    std::vector<SlotState> slot;
    std::vector<std::vector<int>> rows;  // host copy of the table
    // windowed prefill plan (plan_windowed_prefill): text pool shared by all layers, row index arrays
    void* text_k = nullptr;
    void* text_v = nullptr;
    int text_blocks_cap = 0, text_blocks = 0;
    int* d_pf = nullptr;  // [v_slots nv][v_pos nv][t_slots nt][t_pos nt][t_block0 nt][t_len nt]
    int pf_cap = 0, pf_nv = 0, pf_nt = 0;
    std::vector<uocr_b200_prefill_tile> pf_tiles;
    unsigned pf_plan_serial = 0;  // the workspace's plan count after this prefill's plan was made (0: not planned yet)
    int ws_rows = 0;
    // snapshot export: manifest entries written so far, per directory (tensor name -> "file/shape" json)
    std::map<std::string, std::map<std::string, std::string>> manifests;
    std::map<std::string, std::map<std::string, long long>> manifest_ints;

    std::size_t block_bytes() const {
        return static_cast<std::size_t>(cfg.kv_heads) * UOCR_B200_BLOCK_TOKENS * cfg.head_dim *
               (cfg.dtype == DType::BF16 ? 2 : 4);
    }
    void free_all() {
        for (void* p : kpool) if (p) cudaFree(p);
        for (void* p : vpool) if (p) cudaFree(p);
        kpool.clear();
        vpool.clear();
        if (d_table) cudaFree(d_table);
        if (d_len) cudaFree(d_len);
        if (d_ring) cudaFree(d_ring);
        if (d_prefill) cudaFree(d_prefill);
        drop_graphs();
        for (int i = 0; i < 2; ++i) {
            if (d_stage[i]) cudaFree(d_stage[i]);
            if (h_stage[i]) cudaFreeHost(h_stage[i]);
            if (stage_done[i]) cudaEventDestroy(stage_done[i]);
            d_stage[i] = h_stage[i] = nullptr;
            stage_done[i] = nullptr;
            stage_used[i] = false;
        }
        if (text_k) cudaFree(text_k);
        if (text_v) cudaFree(text_v);
        if (d_pf) cudaFree(d_pf);
        text_k = text_v = nullptr;
        d_pf = nullptr;
        text_blocks_cap = text_blocks = pf_cap = pf_nv = pf_nt = 0;
        pf_tiles.clear();
        d_table = nullptr; d_len = d_ring = d_prefill = nullptr;
        if (ws) uocr_b200_workspace_destroy(ws);
        ws = nullptr;
    }
    void drop_graphs() {
        for (auto& kv : step_graphs) {
            if (kv.second.exec) cudaGraphExecDestroy(kv.second.exec);
            if (kv.second.graph) cudaGraphDestroy(kv.second.graph);
        }
        step_graphs.clear();
    }
    int record_ints() const { return 3 + stride; }
    // Brings `n` staged records over with one copy and applies them with one kernel, both on `stream`.
    // `fill(i, rec)` writes record i into pinned memory.  No host synchronisation unless both staging
    // buffers are still being read by earlier copies.
    template <typename Fill>
    void publish(int n, Fill fill, cudaStream_t stream) {
        if (n <= 0) return;
        UOCR_CHECK(n <= cfg.slots, "PagedBatchKV: more slot records than slots");
        const int b = stage_next;
        stage_next ^= 1;
        if (stage_used[b]) cuda_ok(cudaEventSynchronize(stage_done[b]), "slot state staging");
        const int ri = record_ints();
        for (int i = 0; i < n; ++i) fill(i, h_stage[b] + static_cast<std::size_t>(i) * ri);
        cuda_ok(cudaMemcpyAsync(d_stage[b], h_stage[b], sizeof(int) * static_cast<std::size_t>(n) * ri, cudaMemcpyHostToDevice,
                                stream), "slot state H2D");
        cuda_ok(cudaEventRecord(stage_done[b], stream), "slot state event");
        stage_used[b] = true;
        abi_ok(uocr_b200_rswa_publish_slots(d_stage[b], n, d_table, stride, d_len, d_ring, d_prefill, cfg.slots, cfg.layers, ws,
                                            stream), "slot state publication");
    }
    ~Impl() { free_all(); }
};

PagedBatchKV::PagedBatchKV() : p_(new Impl) {}
PagedBatchKV::~PagedBatchKV() = default;
const PagedBatchKV::Config& PagedBatchKV::config() const { return p_->cfg; }
const BlockManager& PagedBatchKV::blocks() const { return *p_->bm; }
const std::vector<int>& PagedBatchKV::table_row(int slot) const { return p_->rows[slot]; }
const uocr_b200_paged_kv& PagedBatchKV::layer_view(int layer) const { return p_->view[layer]; }
int* PagedBatchKV::d_len(int layer) const { return p_->d_len + static_cast<std::size_t>(layer) * p_->cfg.slots; }
int* PagedBatchKV::d_ring_pos(int layer) const { return p_->d_ring + static_cast<std::size_t>(layer) * p_->cfg.slots; }
int* PagedBatchKV::d_prefill_len() const { return p_->d_prefill; }

bool PagedBatchKV::configure(const Config& c) {
    UOCR_CHECK(c.slots > 0 && c.layers > 0 && c.kv_heads > 0 && c.head_dim > 0 && c.window > 0, "PagedBatchKV: bad geometry");
    UOCR_CHECK(c.dtype == DType::BF16 || c.dtype == DType::F32, "PagedBatchKV: dtype must be BF16 or F32");
    UOCR_CHECK(c.ring_arena_blocks >= blocks_for(c.window), "PagedBatchKV: ring arena smaller than one ring");
    Impl& s = *p_;
    const Config& o = s.cfg;
    const bool same = !s.kpool.empty() && o.slots == c.slots && o.layers == c.layers && o.kv_heads == c.kv_heads &&
                      o.head_dim == c.head_dim && o.window == c.window && o.max_prefix_tokens == c.max_prefix_tokens &&
                      o.prefix_arena_blocks == c.prefix_arena_blocks && o.ring_arena_blocks == c.ring_arena_blocks &&
                      o.dtype == c.dtype;
    if (!same) {
        s.free_all();
        s.cfg = c;
        s.stride = blocks_for(c.max_prefix_tokens) + blocks_for(c.window);
        s.num_blocks = c.prefix_arena_blocks + c.ring_arena_blocks;
        s.kpool.assign(static_cast<std::size_t>(c.layers), nullptr);
        s.vpool.assign(static_cast<std::size_t>(c.layers), nullptr);
        const std::size_t bytes = s.block_bytes() * s.num_blocks;
        for (int l = 0; l < c.layers; ++l) {
            cuda_ok(cudaMalloc(&s.kpool[l], bytes), "batch K pool");
            cuda_ok(cudaMalloc(&s.vpool[l], bytes), "batch V pool");
        }
        cuda_ok(cudaMalloc(&s.d_table, sizeof(int32_t) * c.slots * s.stride), "batch table");
        cuda_ok(cudaMalloc(&s.d_len, sizeof(int) * c.layers * c.slots), "batch len");
        cuda_ok(cudaMalloc(&s.d_ring, sizeof(int) * c.layers * c.slots), "batch ring");
        cuda_ok(cudaMalloc(&s.d_prefill, sizeof(int) * c.slots), "batch prefill");
        for (int i = 0; i < 2; ++i) {
            const std::size_t bytes = sizeof(int) * static_cast<std::size_t>(c.slots) * (3 + s.stride);
            cuda_ok(cudaMallocHost(&s.h_stage[i], bytes), "slot state staging (pinned)");
            cuda_ok(cudaMalloc(&s.d_stage[i], bytes), "slot state staging (device)");
            cuda_ok(cudaEventCreateWithFlags(&s.stage_done[i], cudaEventDisableTiming), "slot state event");
        }
        s.ws_rows = std::max(c.slots, 4096);
        abi_ok(uocr_b200_workspace_create(s.ws_rows, &s.ws), "batch workspace");
        s.view.assign(static_cast<std::size_t>(c.layers), uocr_b200_paged_kv{});
        for (int l = 0; l < c.layers; ++l) {
            s.view[l].k_pool = s.kpool[l];
            s.view[l].v_pool = s.vpool[l];
            s.view[l].block_table = s.d_table;
            s.view[l].table_stride = s.stride;
            s.view[l].num_blocks = s.num_blocks;
            s.view[l].kv_heads = c.kv_heads;
            s.view[l].head_dim = c.head_dim;
            s.view[l].dtype = c.dtype == DType::BF16 ? UOCR_B200_BF16 : UOCR_B200_F32;
        }
    }
    // (re)start from an empty state: zero KV and cursors, fresh allocator
    const std::size_t bytes = s.block_bytes() * s.num_blocks;
    for (int l = 0; l < c.layers; ++l) {
        cuda_ok(cudaMemset(s.kpool[l], 0, bytes), "batch K zero");
        cuda_ok(cudaMemset(s.vpool[l], 0, bytes), "batch V zero");
    }
    cuda_ok(cudaMemset(s.d_table, 0xff, sizeof(int32_t) * c.slots * s.stride), "batch table clear");
    cuda_ok(cudaMemset(s.d_len, 0, sizeof(int) * c.layers * c.slots), "batch len zero");
    cuda_ok(cudaMemset(s.d_ring, 0, sizeof(int) * c.layers * c.slots), "batch ring zero");
    cuda_ok(cudaMemset(s.d_prefill, 0, sizeof(int) * c.slots), "batch prefill zero");
    s.bm.reset(new BlockManager(static_cast<std::size_t>(c.prefix_arena_blocks) * 256,
                                static_cast<std::size_t>(c.ring_arena_blocks) * 256));
    s.slot.assign(static_cast<std::size_t>(c.slots), Impl::SlotState{});
    s.rows.assign(static_cast<std::size_t>(c.slots), std::vector<int>(static_cast<std::size_t>(s.stride), -1));
    return !same;
}

void PagedBatchKV::publish_prefill_state(int slot, int prefix_len, cudaStream_t stream) {
    Impl& s = *p_;
    UOCR_CHECK(slot >= 0 && slot < s.cfg.slots, "PagedBatchKV: slot out of range");
    UOCR_CHECK(prefix_len >= 0, "PagedBatchKV: negative prefix length");
    s.publish(1, [&](int, int* rec) {
        rec[0] = slot;
        rec[1] = prefix_len;
        rec[2] = 0;  // the table row stays as it is
    }, stream);
    s.slot[slot].prefix_len = prefix_len;
}

void PagedBatchKV::set_overlap(bool enabled) {
    UOCR_CHECK(p_->ws != nullptr, "PagedBatchKV: not configured");
    abi_ok(uocr_b200_workspace_set_overlap(p_->ws, enabled ? 1 : 0), "set_overlap");
}

std::vector<PagedBatchKV::Admission> PagedBatchKV::admit_wave(const std::vector<WaveItem>& items, cudaStream_t stream) {
    Impl& s = *p_;
    std::vector<Admission> out;
    out.reserve(items.size());
    const int rb = blocks_for(s.cfg.window);
    std::size_t done = 0;
    auto unbind = [&](int slot) {  // host-side undo of one admission of this wave
        Impl::SlotState& st = s.slot[slot];
        s.bm->free_ring(st.ring_off, static_cast<std::size_t>(rb) * 256);
        if (st.has_prefix) s.bm->release_prefix(st.key);
        st = Impl::SlotState{};
        std::fill(s.rows[slot].begin(), s.rows[slot].end(), -1);
    };
    try {
        for (; done < items.size(); ++done) {
            const WaveItem& it = items[done];
            UOCR_CHECK(it.slot >= 0 && it.slot < s.cfg.slots, "PagedBatchKV: slot out of range");
            UOCR_CHECK(!s.slot[it.slot].bound, "PagedBatchKV: slot already bound");
            UOCR_CHECK(it.prefix_len >= 0 && it.prefix_len <= s.cfg.max_prefix_tokens, "PagedBatchKV: prefix longer than configured");
            Admission a;
            a.slot = it.slot;
            const int pb = blocks_for(it.prefix_len);
            std::vector<int>& row = s.rows[it.slot];
            std::fill(row.begin(), row.end(), -1);
            if (pb > 0) {
                const std::size_t live_before = s.bm->live_prefixes();
                PrefixEntry* e = s.bm->acquire_prefix(it.doc_key, it.prefix_len, static_cast<std::size_t>(pb) * 256);  // throws when exhausted
                if (e->prefill_len != it.prefix_len) {
                    s.bm->release_prefix(it.doc_key);
                    UOCR_THROW("PagedBatchKV: doc_key reused with a different prefix length");
                }
                a.prefix_is_new = s.bm->live_prefixes() != live_before;
                a.prefix_refcount = e->refcount;
                for (int i = 0; i < pb; ++i) row[static_cast<std::size_t>(i)] = static_cast<int>(e->offset / 256) + i;
            }
            const i64 roff = s.bm->allocate_ring(static_cast<std::size_t>(rb) * 256);
            if (roff < 0) {
                if (pb > 0) s.bm->release_prefix(it.doc_key);
                std::fill(row.begin(), row.end(), -1);
                UOCR_THROW("ring pool exhausted");
            }
            for (int i = 0; i < rb; ++i)
                row[static_cast<std::size_t>(pb + i)] = s.cfg.prefix_arena_blocks + static_cast<int>(roff / 256) + i;
            Impl::SlotState& st = s.slot[it.slot];
            st.bound = true;
            st.key = it.doc_key;
            st.has_prefix = pb > 0;
            st.ring_off = roff;
            st.prefix_len = it.prefix_len;
            out.push_back(a);
        }
    } catch (...) {
        for (std::size_t i = 0; i < done; ++i) unbind(items[i].slot);
        throw;
    }
    s.publish(static_cast<int>(items.size()), [&](int i, int* rec) {
        rec[0] = items[static_cast<std::size_t>(i)].slot;
        rec[1] = items[static_cast<std::size_t>(i)].prefix_len;
        rec[2] = 1;
        std::memcpy(rec + 3, s.rows[items[static_cast<std::size_t>(i)].slot].data(), sizeof(int) * s.stride);
    }, stream);
    return out;
}

PagedBatchKV::Admission PagedBatchKV::admit(int slot, const std::string& doc_key, int prefix_len, cudaStream_t stream) {
    return admit_wave({WaveItem{slot, doc_key, prefix_len}}, stream)[0];
}

void PagedBatchKV::release(int slot, cudaStream_t stream) {
    Impl& s = *p_;
    UOCR_CHECK(slot >= 0 && slot < s.cfg.slots, "PagedBatchKV: slot out of range");
    Impl::SlotState& st = s.slot[slot];
    if (!st.bound) return;
    s.bm->free_ring(st.ring_off, static_cast<std::size_t>(blocks_for(s.cfg.window)) * 256);
    if (st.has_prefix) s.bm->release_prefix(st.key);
    st = Impl::SlotState{};
    std::fill(s.rows[slot].begin(), s.rows[slot].end(), -1);
    s.publish(1, [&](int, int* rec) {  // device row <- -1, cursors <- 0: stale use is flagged, not obeyed
        rec[0] = slot;
        rec[1] = 0;
        rec[2] = 1;
        std::fill(rec + 3, rec + 3 + s.stride, -1);
    }, stream);
}

bool PagedBatchKV::capture_step(int batch, const StepIO& io, cudaStream_t stream) {
    Impl& s = *p_;
    UOCR_CHECK(batch > 0 && batch <= s.cfg.slots, "capture_step: invalid batch size");
    UOCR_CHECK(io.q && io.k && io.v && io.out && io.d_slots && io.heads > 0, "capture_step: incomplete buffer description");
    UOCR_CHECK(stream != nullptr, "capture_step: needs a stream of its own (the legacy default stream cannot be captured)");
    auto it = s.step_graphs.find(batch);
    if (it != s.step_graphs.end()) {
        const StepIO& o = it->second.io;
        const bool same = o.q == io.q && o.k == io.k && o.v == io.v && o.out == io.out && o.d_slots == io.d_slots &&
                          o.q_layer_stride == io.q_layer_stride && o.kv_layer_stride == io.kv_layer_stride &&
                          o.out_layer_stride == io.out_layer_stride && o.heads == io.heads && o.d_positions == io.d_positions &&
                          o.rope_theta == io.rope_theta;
        if (same) return false;
        cudaGraphExecDestroy(it->second.exec);
        cudaGraphDestroy(it->second.graph);
        s.step_graphs.erase(it);
    }
    Impl::StepGraph g;
    g.io = io;
    cuda_ok(cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal), "begin step capture");
    try {
        for (int l = 0; l < s.cfg.layers; ++l) {
            const float* q = io.q + static_cast<std::size_t>(l) * io.q_layer_stride;
            const float* k = io.k + static_cast<std::size_t>(l) * io.kv_layer_stride;
            const float* v = io.v + static_cast<std::size_t>(l) * io.kv_layer_stride;
            float* out = io.out + static_cast<std::size_t>(l) * io.out_layer_stride;
            if (io.d_positions)
                decode_step_rope(l, q, k, v, io.d_positions, io.rope_theta, io.d_slots, batch, io.heads, out, stream);
            else
                decode_step(l, q, k, v, io.d_slots, batch, io.heads, out, stream);
        }
    } catch (...) {
        cudaGraph_t broken = nullptr;
        cudaStreamEndCapture(stream, &broken);
        if (broken) cudaGraphDestroy(broken);
        throw;
    }
    cuda_ok(cudaStreamEndCapture(stream, &g.graph), "end step capture");
    cuda_ok(cudaGraphInstantiate(&g.exec, g.graph, nullptr, nullptr, 0), "instantiate step graph");
    s.step_graphs[batch] = g;
    return true;
}

void PagedBatchKV::replay_step(int batch, cudaStream_t stream) {
    auto it = p_->step_graphs.find(batch);
    UOCR_CHECK(it != p_->step_graphs.end(), "replay_step: no graph captured for this batch size");
    cuda_ok(cudaGraphLaunch(it->second.exec, stream), "step graph launch");
}

int PagedBatchKV::step_graph_count() const { return static_cast<int>(p_->step_graphs.size()); }
void PagedBatchKV::drop_step_graphs() { p_->drop_graphs(); }

void PagedBatchKV::append_decode_batch(int layer, const float* k, const float* v, const int* d_slots, int batch,
                                       cudaStream_t stream) {
    Impl& s = *p_;
    UOCR_CHECK(batch <= s.cfg.slots, "batch_decode size out of range");
    abi_ok(uocr_b200_rswa_append_decode_batch_paged(&s.view[layer], k, v, d_len(layer), d_ring_pos(layer), s.d_prefill,
                                                    d_slots, batch, s.cfg.window, s.ws, stream), "append_decode_batch");
}
void PagedBatchKV::attention_batch(int layer, const float* q, const int* d_slots, int batch, int heads, float* out,
                                   cudaStream_t stream) {
    Impl& s = *p_;
    UOCR_CHECK(batch <= s.cfg.slots, "batch_decode size out of range");
    abi_ok(uocr_b200_rswa_attention_batch_paged(&s.view[layer], q, d_len(layer), s.d_prefill, d_slots, batch, heads, out,
                                                s.ws, stream), "attention_batch");
}
void PagedBatchKV::decode_step(int layer, const float* q, const float* k, const float* v, const int* d_slots, int batch,
                               int heads, float* out, cudaStream_t stream) {
    Impl& s = *p_;
    UOCR_CHECK(batch <= s.cfg.slots, "batch_decode size out of range");
    abi_ok(uocr_b200_rswa_decode_step_paged(&s.view[layer], q, k, v, d_len(layer), d_ring_pos(layer), s.d_prefill, d_slots,
                                            batch, s.cfg.window, heads, out, s.ws, stream), "decode_step");
}
void PagedBatchKV::decode_step_rope(int layer, const float* q, const float* k, const float* v, const int* d_positions,
                                    float theta, const int* d_slots, int batch, int heads, float* out, cudaStream_t stream) {
    Impl& s = *p_;
    UOCR_CHECK(batch <= s.cfg.slots, "batch_decode size out of range");
    abi_ok(uocr_b200_rswa_decode_step_rope_paged(&s.view[layer], q, k, v, d_positions, theta, d_len(layer), d_ring_pos(layer),
                                                 s.d_prefill, d_slots, batch, s.cfg.window, heads, out, s.ws, stream),
           "decode_step_rope");
}
void PagedBatchKV::write_prefill_ragged(int layer, const float* k, const float* v, const int* d_row_slots,
                                        const int* d_pos, int total, cudaStream_t stream) {
    Impl& s = *p_;
    abi_ok(uocr_b200_rswa_write_prefill_ragged_paged(&s.view[layer], k, v, d_row_slots, d_pos, total, s.ws, stream),
           "write_prefill_ragged");
}
int PagedBatchKV::plan_windowed_prefill(const std::vector<WindowedPrefill>& reqs, cudaStream_t stream) {
    Impl& s = *p_;
    int nv = 0, nt = 0, blocks = 0;
    for (const WindowedPrefill& r : reqs) {
        UOCR_CHECK(r.slot >= 0 && r.slot < s.cfg.slots && s.slot[r.slot].bound, "windowed prefill: slot not admitted");
        UOCR_CHECK(r.vision_rows == 0 || r.vision_rows == s.slot[r.slot].prefix_len,
                   "windowed prefill: vision rows must be the slot's whole prefix, or 0 when it is resident");
        UOCR_CHECK(r.text_rows >= 0, "windowed prefill: negative text length");
        nv += r.vision_rows;
        nt += r.text_rows;
        blocks += blocks_for(r.text_rows);
    }
    std::vector<int> idx(static_cast<std::size_t>(2 * nv + 4 * nt));
    int* v_slots = idx.data();
    int* v_pos = v_slots + nv;
    int* t_slots = v_pos + nv;
    int* t_pos = t_slots + nt;
    int* t_b0 = t_pos + nt;
    int* t_len = t_b0 + nt;
    s.pf_tiles.clear();
    s.pf_plan_serial = 0;
    auto add_tiles = [&](int row0, int n, int slot, int kind, int block0) {
        for (int a = 0; a < n; a += 128) s.pf_tiles.push_back({row0 + a, std::min(128, n - a), slot, kind, a, block0});
    };
    int at = 0;
    for (const WindowedPrefill& r : reqs) {
        for (int i = 0; i < r.vision_rows; ++i) {
            v_slots[at + i] = r.slot;
            v_pos[at + i] = i;
        }
        add_tiles(at, r.vision_rows, r.slot, 0, 0);
        at += r.vision_rows;
    }
    int tt = 0, b0 = 0;
    for (const WindowedPrefill& r : reqs) {
        for (int i = 0; i < r.text_rows; ++i) {
            t_slots[tt + i] = r.slot;
            t_pos[tt + i] = i;
            t_b0[tt + i] = b0;
            t_len[tt + i] = r.text_rows;
        }
        add_tiles(nv + tt, r.text_rows, r.slot, 1, b0);
        tt += r.text_rows;
        b0 += blocks_for(r.text_rows);
    }
    UOCR_CHECK(static_cast<int>(s.pf_tiles.size()) <= s.ws_rows, "windowed prefill: more query tiles than the workspace holds");
    if (blocks > s.text_blocks_cap) {  // finite contents everywhere: rows past a request's last token are read, masked
        if (s.text_k) cudaFree(s.text_k);
        if (s.text_v) cudaFree(s.text_v);
        s.text_k = s.text_v = nullptr;
        const std::size_t bytes = s.block_bytes() * static_cast<std::size_t>(blocks);
        cuda_ok(cudaMalloc(&s.text_k, bytes), "text K pool");
        cuda_ok(cudaMalloc(&s.text_v, bytes), "text V pool");
        cuda_ok(cudaMemset(s.text_k, 0, bytes), "text K zero");
        cuda_ok(cudaMemset(s.text_v, 0, bytes), "text V zero");
        s.text_blocks_cap = blocks;
    }
    if (static_cast<int>(idx.size()) > s.pf_cap) {
        if (s.d_pf) cudaFree(s.d_pf);
        s.d_pf = nullptr;
        cuda_ok(cudaMalloc(&s.d_pf, sizeof(int) * idx.size()), "prefill index arrays");
        s.pf_cap = static_cast<int>(idx.size());
    }
    if (!idx.empty()) {
        cuda_ok(cudaMemcpyAsync(s.d_pf, idx.data(), sizeof(int) * idx.size(), cudaMemcpyHostToDevice, stream), "prefill index H2D");
        cuda_ok(cudaStreamSynchronize(stream), "prefill index sync");  // idx is a local
    }
    s.pf_nv = nv;
    s.pf_nt = nt;
    s.text_blocks = blocks;
    return nv + nt;
}

void PagedBatchKV::windowed_prefill_layer(int layer, const float* q, const float* k, const float* v, int heads, float* out,
                                          cudaStream_t stream) {
    Impl& s = *p_;
    const int nv = s.pf_nv, nt = s.pf_nt;
    if (nv + nt == 0) return;
    const uocr_b200_paged_kv* view = &s.view[layer];
    const int row = s.cfg.kv_heads * s.cfg.head_dim, qrow = heads * s.cfg.head_dim;
    const int* v_slots = s.d_pf;
    const int* v_pos = v_slots + nv;
    const int* t_slots = v_pos + nv;
    const int* t_pos = t_slots + nt;
    const int* t_b0 = t_pos + nt;
    const int* t_len = t_b0 + nt;
    const float* kt = k + static_cast<std::size_t>(nv) * row;
    const float* vt = v + static_cast<std::size_t>(nv) * row;
    if (nv > 0)
        abi_ok(uocr_b200_rswa_write_prefill_ragged_paged(view, k, v, v_slots, v_pos, nv, s.ws, stream), "windowed prefill: prefix scatter");
    const bool tensor_cores = s.cfg.dtype == DType::BF16 && s.cfg.head_dim == 128;
    if (tensor_cores) {
        if (nt > 0)  // text pool, ring blocks and cursors in one pass; the attention below reads none of the latter two
            abi_ok(uocr_b200_rswa_text_scatter_fill_paged(view, s.text_k, s.text_v, s.text_blocks, kt, vt, t_slots, t_pos, t_b0, t_len,
                                                          s.d_prefill, d_len(layer), d_ring_pos(layer), nt, s.cfg.window, s.ws, stream),
                   "windowed prefill: text scatter + ring fill");
        // the layers of one prefill share one plan of the query tiles (made by the first call, reused while it is
        // still the workspace's last)
        const bool planned = s.pf_plan_serial != 0 && s.pf_plan_serial == uocr_b200_workspace_prefill_plan_serial(s.ws);
        abi_ok(uocr_b200_rswa_prefill_attention_tc(view, s.text_k, s.text_v, s.text_blocks, q, s.d_prefill,
                                                   planned ? nullptr : s.pf_tiles.data(), static_cast<int>(s.pf_tiles.size()),
                                                   s.cfg.window, heads, out, s.ws, stream),
               "windowed prefill: attention");
        s.pf_plan_serial = uocr_b200_workspace_prefill_plan_serial(s.ws);
    } else {
        for (int a = 0; a < nv; a += s.ws_rows) {  // the split-KV scratch holds ws_rows query rows per call
            const int n = std::min(s.ws_rows, nv - a);
            abi_ok(uocr_b200_rswa_attention_ragged_paged(view, q + static_cast<std::size_t>(a) * qrow, s.d_prefill, v_slots + a,
                                                         v_pos + a, n, heads, out + static_cast<std::size_t>(a) * qrow, s.ws, stream),
                   "windowed prefill: vision attention");
        }
        for (int a = 0; a < nt; a += s.ws_rows) {
            const int n = std::min(s.ws_rows, nt - a);
            const std::size_t r0 = static_cast<std::size_t>(nv + a);
            abi_ok(uocr_b200_rswa_prefill_text_paged(view, s.text_k, s.text_v, s.text_blocks, q + r0 * qrow,
                                                     kt + static_cast<std::size_t>(a) * row, vt + static_cast<std::size_t>(a) * row,
                                                     s.d_prefill, t_slots + a, t_pos + a, t_b0 + a, n, s.cfg.window, heads,
                                                     out + r0 * qrow, s.ws, stream),
                   "windowed prefill: text attention");
        }
    }
    if (nt > 0 && !tensor_cores)
        abi_ok(uocr_b200_rswa_ring_fill_paged(view, s.text_k, s.text_v, s.text_blocks, t_slots, t_pos, t_b0, t_len, s.d_prefill,
                                              d_len(layer), d_ring_pos(layer), nt, s.cfg.window, s.ws, stream),
               "windowed prefill: ring fill");
}

void PagedBatchKV::export_snapshot(const std::string& dir, int slot, const std::string& tag, cudaStream_t stream) {
    Impl& s = *p_;
    UOCR_CHECK(slot >= 0 && slot < s.cfg.slots && s.slot[slot].bound, "export_snapshot: slot not admitted");
    UOCR_CHECK(tag == "prefill" || tag == "final", "export_snapshot: tag must be \"prefill\" or \"final\"");
    const int cap = s.cfg.max_prefix_tokens + s.cfg.window, kvh = s.cfg.kv_heads, hd = s.cfg.head_dim;
    const std::size_t elems = static_cast<std::size_t>(kvh) * cap * hd;
    float *dk = nullptr, *dv = nullptr;
    int* d_slot = nullptr;
    cuda_ok(cudaMalloc(&dk, elems * sizeof(float)), "snapshot K buffer");
    cudaError_t e = cudaMalloc(&dv, elems * sizeof(float));
    if (e == cudaSuccess) e = cudaMalloc(&d_slot, sizeof(int));
    std::vector<float> hk(elems), hv(elems);
    std::vector<int> lens(static_cast<std::size_t>(s.cfg.layers), 0);
    std::string err;
    auto write_bin = [&](const std::string& name, const std::vector<float>& full, int len) {
        // full is [kvh][cap][hd]; the file keeps the first `len` rows of every head
        FILE* f = std::fopen((dir + "/" + name + ".bin").c_str(), "wb");
        if (!f) { err = "cannot write " + dir + "/" + name + ".bin"; return; }
        for (int h = 0; h < kvh && err.empty(); ++h)
            if (len > 0 && std::fwrite(full.data() + static_cast<std::size_t>(h) * cap * hd, sizeof(float),
                                       static_cast<std::size_t>(len) * hd, f) != static_cast<std::size_t>(len) * hd)
                err = "short write to " + dir + "/" + name + ".bin";
        std::fclose(f);
        s.manifests[dir][name] = "{\"file\": \"" + name + ".bin\", \"shape\": [" + std::to_string(kvh) + ", " +
                                 std::to_string(len) + ", " + std::to_string(hd) + "], \"dtype\": \"<f4\"}";
    };
    if (e == cudaSuccess) e = cudaMemcpyAsync(d_slot, &slot, sizeof(int), cudaMemcpyHostToDevice, stream);
    if (e == cudaSuccess) e = cudaMemcpy2DAsync(lens.data(), sizeof(int), s.d_len + slot, sizeof(int) * s.cfg.slots, sizeof(int),
                                                s.cfg.layers, cudaMemcpyDeviceToHost, stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
    for (int l = 0; l < s.cfg.layers && e == cudaSuccess && err.empty(); ++l) {
        const int rc = uocr_b200_rswa_gather_heads_paged(&s.view[l], d_len(l), s.d_prefill, d_slot, 1, cap, dk, dv, s.ws, stream);
        if (rc != UOCR_B200_OK) { err = std::string("gather: ") + uocr_b200_last_error(); break; }
        e = cudaMemcpyAsync(hk.data(), dk, elems * sizeof(float), cudaMemcpyDeviceToHost, stream);
        if (e == cudaSuccess) e = cudaMemcpyAsync(hv.data(), dv, elems * sizeof(float), cudaMemcpyDeviceToHost, stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
        if (e != cudaSuccess) break;
        write_bin(tag + "_k_" + std::to_string(l), hk, lens[l]);
        if (err.empty()) write_bin(tag + "_v_" + std::to_string(l), hv, lens[l]);
    }
    cudaFree(dk);
    if (dv) cudaFree(dv);
    if (d_slot) cudaFree(d_slot);
    cuda_ok(e, "export_snapshot");
    if (!err.empty()) UOCR_THROW("export_snapshot: " + err);
    auto& ints = s.manifest_ints[dir];
    ints["window"] = s.cfg.window;
    ints["cache_layers"] = s.cfg.layers;
    ints["kv_heads"] = kvh;
    ints["head_dim"] = hd;
    ints[tag + "_cache_len"] = lens[0];
    FILE* f = std::fopen((dir + "/manifest.json").c_str(), "w");
    if (!f) UOCR_THROW("export_snapshot: cannot write " + dir + "/manifest.json");
    std::fprintf(f, "{\n");
    for (const auto& kv : ints) std::fprintf(f, "  \"%s\": %lld,\n", kv.first.c_str(), kv.second);
    std::fprintf(f, "  \"tensors\": {\n");
    std::size_t i = 0;
    const auto& tensors = s.manifests[dir];
    for (const auto& kv : tensors)
        std::fprintf(f, "    \"%s\": %s%s\n", kv.first.c_str(), kv.second.c_str(), ++i < tensors.size() ? "," : "");
    std::fprintf(f, "  }\n}\n");
    std::fclose(f);
}

void PagedBatchKV::attention_ragged(int layer, const float* q, const int* d_row_slots, const int* d_pos, int total,
                                    int heads, float* out, cudaStream_t stream) {
    Impl& s = *p_;
    const std::size_t qrow = static_cast<std::size_t>(heads) * s.cfg.head_dim;
    for (int a = 0; a < total; a += s.ws_rows) {  // the split-KV scratch holds ws_rows query rows per call; rows are independent
        const int n = std::min(s.ws_rows, total - a);
        abi_ok(uocr_b200_rswa_attention_ragged_paged(&s.view[layer], q + a * qrow, s.d_prefill, d_row_slots + a, d_pos + a, n,
                                                     heads, out + a * qrow, s.ws, stream), "attention_ragged");
    }
}
void PagedBatchKV::gather(int layer, const int* d_slots, int n, float* out_k, float* out_v, cudaStream_t stream) {
    Impl& s = *p_;
    abi_ok(uocr_b200_rswa_gather_paged(&s.view[layer], d_len(layer), s.d_prefill, d_slots, n,
                                       s.cfg.max_prefix_tokens + s.cfg.window, out_k, out_v, UOCR_B200_F32, s.ws, stream),
           "gather");
}
int PagedBatchKV::device_status(cudaStream_t stream) {
    int v = 0;
    abi_ok(uocr_b200_workspace_status(p_->ws, stream, &v), "device_status");
    return v;
}

// =================================================================================================
// GpuDecoderKV -- KV half of GpuDecoder's continuous-batching interface (gpu_decoder.h:69-87)
// =================================================================================================
struct GpuDecoderKV::Impl {
    int layers = 0, kv_heads = 0, head_dim = 0, window = 0;
    DType dtype = DType::BF16;
    PagedBatchKV kv;
    int slots = 0, capacity = 0;
    int* d_batch_slots = nullptr;  // [slots] row -> slot of the current decode batch
    int* d_positions = nullptr;    // [slots] positions of the current decode batch (rotary step only)
    int* d_row_slot = nullptr;     // ragged prefill: [packed row -> slot][packed row -> position inside its request]
    int ragged_cap = 0;            // packed rows the array above holds (it is 2 * ragged_cap ints long)
    unsigned long long anon = 0;   // requests without a doc_key get a key of their own

    void free_index_arrays() {
        for (int** p : {&d_batch_slots, &d_positions, &d_row_slot}) {
            if (*p) cudaFree(*p);
            *p = nullptr;
        }
        ragged_cap = 0;
    }
    ~Impl() { free_index_arrays(); }
};

GpuDecoderKV::GpuDecoderKV(int num_layers, int kv_heads, int head_dim, int window, DType dtype) : p_(new Impl) {
    UOCR_CHECK(num_layers > 0 && kv_heads > 0 && head_dim > 0 && window > 0, "GpuDecoderKV: bad geometry");
    p_->layers = num_layers;
    p_->kv_heads = kv_heads;
    p_->head_dim = head_dim;
    p_->window = window;
    p_->dtype = dtype;
}
GpuDecoderKV::~GpuDecoderKV() = default;
PagedBatchKV& GpuDecoderKV::kv() { return p_->kv; }
int GpuDecoderKV::batch_slots() const { return p_->slots; }
int GpuDecoderKV::batch_graph_count() const { return p_->slots ? p_->kv.step_graph_count() : 0; }
const int* GpuDecoderKV::d_batch_slots() const { return p_->d_batch_slots; }

bool GpuDecoderKV::batch_configure(int slots, int capacity) {
    Impl& s = *p_;
    UOCR_CHECK(slots > 0 && capacity > s.window, "batch_configure: invalid shape");
    PagedBatchKV::Config c;
    c.slots = slots;
    c.layers = s.layers;
    c.kv_heads = s.kv_heads;
    c.head_dim = s.head_dim;
    c.window = s.window;
    c.dtype = s.dtype;
    c.max_prefix_tokens = capacity - s.window;  // the reference sizes every slot for the longest prompt + window
    c.prefix_arena_blocks = slots * blocks_for(c.max_prefix_tokens);  // worst case: no two requests share a prefix
    c.ring_arena_blocks = slots * blocks_for(s.window);
    const bool fresh = s.kv.configure(c);
    if (fresh || slots != s.slots) {
        s.free_index_arrays();
        cuda_ok(cudaMalloc(&s.d_batch_slots, sizeof(int) * slots), "batch slots");
        cuda_ok(cudaMalloc(&s.d_positions, sizeof(int) * slots), "batch positions");
    }
    s.slots = slots;
    s.capacity = capacity;
    return fresh;
}

int GpuDecoderKV::batch_prefill_begin(const std::vector<int>& starts, const std::vector<int>& lengths,
                                      const std::vector<int>& slots, const std::vector<std::string>& doc_keys,
                                      cudaStream_t stream) {
    Impl& s = *p_;
    const int requests = static_cast<int>(lengths.size());
    UOCR_CHECK(requests > 0, "batch_prefill_embeds: no requests");
    UOCR_CHECK(static_cast<int>(starts.size()) == requests && static_cast<int>(slots.size()) == requests,
               "batch_prefill_embeds: array size mismatch");
    UOCR_CHECK(doc_keys.empty() || static_cast<int>(doc_keys.size()) == requests, "batch_prefill_embeds: doc_keys size mismatch");
    int total = 0;
    std::vector<PagedBatchKV::WaveItem> wave;
    for (int r = 0; r < requests; ++r) {
        UOCR_CHECK(lengths[r] > 0, "batch_prefill_embeds: empty prompt");
        UOCR_CHECK(starts[r] == total, "batch_prefill_embeds: non-contiguous starts");
        UOCR_CHECK(slots[r] >= 0 && slots[r] < s.slots, "batch_prefill_embeds: slot out of range");
        total += lengths[r];
        const std::string key = (!doc_keys.empty() && !doc_keys[r].empty()) ? doc_keys[r] : "#request" + std::to_string(s.anon++);
        wave.push_back({slots[r], key, lengths[r]});
    }
    s.kv.admit_wave(wave, stream);  // table rows + len = prefill = prompt length, ring_pos = 0: one upload
    std::vector<int> idx(static_cast<std::size_t>(2 * total));
    for (int r = 0; r < requests; ++r)
        for (int p = 0; p < lengths[r]; ++p) {
            idx[static_cast<std::size_t>(starts[r] + p)] = slots[r];
            idx[static_cast<std::size_t>(total + starts[r] + p)] = p;
        }
    if (total > s.ragged_cap) {
        if (s.d_row_slot) cudaFree(s.d_row_slot);
        s.d_row_slot = nullptr;
        cuda_ok(cudaMalloc(&s.d_row_slot, sizeof(int) * 2 * static_cast<std::size_t>(total)), "ragged row index");
        s.ragged_cap = total;
    }
    // pageable source: the copy has staged `idx` when the call returns
    cuda_ok(cudaMemcpyAsync(s.d_row_slot, idx.data(), sizeof(int) * idx.size(), cudaMemcpyHostToDevice, stream), "ragged index H2D");
    return total;
}

void GpuDecoderKV::attention_block_ragged(int li, const float* q, const float* k, const float* v, float* ctx, int total,
                                          int heads, cudaStream_t stream) {
    Impl& s = *p_;
    UOCR_CHECK(s.d_row_slot != nullptr && total > 0 && total <= s.ragged_cap, "attention_block_ragged: call batch_prefill_begin first");
    const int* row_slot = s.d_row_slot;
    const int* row_pos = s.d_row_slot + total;  // second half of the array staged by batch_prefill_begin
    s.kv.write_prefill_ragged(li, k, v, row_slot, row_pos, total, stream);
    s.kv.attention_ragged(li, q, row_slot, row_pos, total, heads, ctx, stream);
}

void GpuDecoderKV::batch_decode_begin(const std::vector<int>& slots, cudaStream_t stream) {
    Impl& s = *p_;
    const int batch = static_cast<int>(slots.size());
    UOCR_CHECK(batch > 0 && batch <= s.slots, "batch_decode size out of range");
    cuda_ok(cudaMemcpyAsync(s.d_batch_slots, slots.data(), sizeof(int) * batch, cudaMemcpyHostToDevice, stream), "batch slots");
}

void GpuDecoderKV::attention_block_batch(int li, const float* q, const float* k, const float* v, float* ctx, int batch,
                                         int heads, cudaStream_t stream) {
    Impl& s = *p_;
    UOCR_CHECK(batch > 0 && batch <= s.slots, "batch_decode size out of range");
    s.kv.decode_step(li, q, k, v, s.d_batch_slots, batch, heads, ctx, stream);  // append + attention, one launch
}

void GpuDecoderKV::batch_decode(const std::vector<int>& positions, const std::vector<int>& slots,
                                const PagedBatchKV::StepIO& io, bool fold_rope, cudaStream_t stream) {
    Impl& s = *p_;
    const int batch = static_cast<int>(slots.size());
    UOCR_CHECK(batch > 0 && batch <= s.slots, "batch_decode size out of range");
    UOCR_CHECK(!fold_rope || static_cast<int>(positions.size()) == batch, "positions size mismatch");
    cuda_ok(cudaMemcpyAsync(s.d_batch_slots, slots.data(), sizeof(int) * batch, cudaMemcpyHostToDevice, stream), "batch slots");
    if (fold_rope)
        cuda_ok(cudaMemcpyAsync(s.d_positions, positions.data(), sizeof(int) * batch, cudaMemcpyHostToDevice, stream), "batch pos");
    PagedBatchKV::StepIO fixed = io;
    fixed.d_slots = s.d_batch_slots;
    fixed.d_positions = fold_rope ? s.d_positions : nullptr;
    s.kv.capture_step(batch, fixed, stream);  // no-op when this batch size was captured on these buffers
    s.kv.replay_step(batch, stream);
}

void GpuDecoderKV::batch_release(int slot, cudaStream_t stream) { p_->kv.release(slot, stream); }

}  // namespace cuda
}  // namespace uocr
