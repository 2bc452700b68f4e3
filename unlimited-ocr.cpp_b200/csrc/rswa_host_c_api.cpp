// extern "C" wrappers over the host-side classes (include/uocr_rswa_b200_host.h).
#include "uocr_rswa_b200_host.h"

#include <string>

#include "uocr/rswa_host.h"

using namespace uocr;

namespace {
thread_local std::string g_host_error;
template <typename F>
int guarded(F&& f) {
    try {
        f();
        return 0;
    } catch (const std::exception& e) {
        g_host_error = e.what();
        return -1;
    }
}
}  // namespace

extern "C" {

// ---- MemoryPool ------------------------------------------------------------------------------------
void* uocr_b200_pool_create(size_t bytes, size_t alignment) { return new MemoryPool(bytes, alignment); }
void uocr_b200_pool_destroy(void* p) { delete static_cast<MemoryPool*>(p); }
void uocr_b200_pool_reset(void* p) { static_cast<MemoryPool*>(p)->reset(); }
int64_t uocr_b200_pool_allocate(void* p, size_t bytes, size_t alignment) { return static_cast<MemoryPool*>(p)->allocate(bytes, alignment); }
void uocr_b200_pool_free(void* p, int64_t off, size_t bytes) { static_cast<MemoryPool*>(p)->free(off, bytes); }
size_t uocr_b200_pool_total(const void* p) { return static_cast<const MemoryPool*>(p)->total(); }
size_t uocr_b200_pool_used(const void* p) { return static_cast<const MemoryPool*>(p)->used(); }
size_t uocr_b200_pool_peak(const void* p) { return static_cast<const MemoryPool*>(p)->peak(); }
size_t uocr_b200_pool_num_free_blocks(const void* p) { return static_cast<const MemoryPool*>(p)->num_free_blocks(); }
double uocr_b200_pool_fragmentation(const void* p) { return static_cast<const MemoryPool*>(p)->fragmentation(); }

// ---- BlockManager -----------------------------------------------------------------------------------
void* uocr_b200_bm_create(size_t prefix_bytes, size_t ring_bytes) { return new BlockManager(prefix_bytes, ring_bytes); }
void uocr_b200_bm_destroy(void* m) { delete static_cast<BlockManager*>(m); }
int64_t uocr_b200_bm_acquire_prefix(void* m, const char* key, int prefill_len, size_t bytes, int* refcount) {
    int64_t off = -1;
    if (guarded([&] {
            PrefixEntry* e = static_cast<BlockManager*>(m)->acquire_prefix(key, prefill_len, bytes);
            off = e->offset;
            if (refcount) *refcount = e->refcount;
        }) != 0)
        return -1;
    return off;
}
void uocr_b200_bm_release_prefix(void* m, const char* key) { static_cast<BlockManager*>(m)->release_prefix(key); }
int64_t uocr_b200_bm_allocate_ring(void* m, size_t bytes) { return static_cast<BlockManager*>(m)->allocate_ring(bytes); }
void uocr_b200_bm_free_ring(void* m, int64_t off, size_t bytes) { static_cast<BlockManager*>(m)->free_ring(off, bytes); }
uint64_t uocr_b200_bm_live_prefixes(const void* m) { return static_cast<const BlockManager*>(m)->live_prefixes(); }
uint64_t uocr_b200_bm_total_prefix_bytes(const void* m) { return static_cast<const BlockManager*>(m)->total_prefix_bytes(); }
uint64_t uocr_b200_bm_shared_prefix_bytes(const void* m) { return static_cast<const BlockManager*>(m)->shared_prefix_bytes(); }
uint64_t uocr_b200_bm_peak_prefix_bytes(const void* m) { return static_cast<const BlockManager*>(m)->peak_prefix_bytes(); }
void uocr_b200_bm_get_stats(const void* m, uocr_b200_bm_stats* o) {
    const BlockManager::Stats s = static_cast<const BlockManager*>(m)->stats();
    o->prefix_live_bytes = s.prefix_live_bytes;
    o->prefix_peak_bytes = s.prefix_peak_bytes;
    o->prefix_shared_bytes = s.prefix_shared_bytes;
    o->ring_live_bytes = s.ring_live_bytes;
    o->ring_peak_bytes = s.ring_peak_bytes;
    o->prefix_fragmentation = s.prefix_fragmentation;
    o->ring_fragmentation = s.ring_fragmentation;
    o->live_prefixes = s.live_prefixes;
}

// ---- ContinuousBatchScheduler --------------------------------------------------------------------------
void* uocr_b200_sched_create(int max_batch, int min_batch) { return new ContinuousBatchScheduler(max_batch, min_batch); }
void uocr_b200_sched_destroy(void* s) { delete static_cast<ContinuousBatchScheduler*>(s); }
int uocr_b200_sched_add_request(void* s, int prompt_len, int max_new_tokens) {
    Request r;
    r.prompt_tokens.assign(static_cast<size_t>(prompt_len), 1);
    r.max_new_tokens = max_new_tokens;
    return static_cast<ContinuousBatchScheduler*>(s)->add_request(std::move(r));
}
void uocr_b200_sched_build_batch(void* s, int* prefill_ids, int* n_prefill, int* decode_ids, int* n_decode, int cap) {
    const Batch b = static_cast<ContinuousBatchScheduler*>(s)->build_batch();
    int np = 0, nd = 0;
    for (int id : b.prefill) if (np < cap) prefill_ids[np++] = id;
    for (int id : b.decode) if (nd < cap) decode_ids[nd++] = id;
    *n_prefill = np;
    *n_decode = nd;
}
void uocr_b200_sched_mark_prefilled(void* s, int id) { static_cast<ContinuousBatchScheduler*>(s)->mark_prefilled(id); }
void uocr_b200_sched_mark_prefilling(void* s, int id) { static_cast<ContinuousBatchScheduler*>(s)->mark_prefilling(id); }
int uocr_b200_sched_add_token(void* s, int id, int token) { return static_cast<ContinuousBatchScheduler*>(s)->add_token(id, token) ? 1 : 0; }
void uocr_b200_sched_finish(void* s, int id) { static_cast<ContinuousBatchScheduler*>(s)->finish(id); }
int uocr_b200_sched_state(const void* s, int id) {
    const Request* r = static_cast<const ContinuousBatchScheduler*>(s)->get(id);
    return r ? static_cast<int>(r->state) : -1;
}
int uocr_b200_sched_num_outputs(const void* s, int id) {
    const Request* r = static_cast<const ContinuousBatchScheduler*>(s)->get(id);
    return r ? static_cast<int>(r->output_tokens.size()) : -1;
}
int uocr_b200_sched_has_work(const void* s) { return static_cast<const ContinuousBatchScheduler*>(s)->has_work() ? 1 : 0; }
int uocr_b200_sched_running(const void* s, int* ids, int cap) {
    const std::vector<int>& r = static_cast<const ContinuousBatchScheduler*>(s)->running();
    for (size_t i = 0; i < r.size() && static_cast<int>(i) < cap; ++i) ids[i] = r[i];
    return static_cast<int>(r.size());
}
void uocr_b200_sched_get_stats(const void* s, uocr_b200_sched_stats* o) {
    const auto st = static_cast<const ContinuousBatchScheduler*>(s)->stats();
    o->total_requests = st.total_requests;
    o->finished_requests = st.finished_requests;
    o->prefill_tokens = st.prefill_tokens;
    o->decode_tokens = st.decode_tokens;
    o->waiting = st.waiting;
    o->running = st.running;
    o->last_batch_size = st.last_batch_size;
}

// ---- RSWACache -------------------------------------------------------------------------------------------
void* uocr_b200_cache_create(int layers, int kv_heads, int head_dim, int window) {
    return new RSWACache(layers, kv_heads, head_dim, window);
}
int uocr_b200_cache_set_kv_dtype(void* c, int dtype) {
    return guarded([&] { static_cast<RSWACache*>(c)->set_kv_dtype(dtype == UOCR_B200_BF16 ? DType::BF16 : DType::F32); });
}
void uocr_b200_cache_destroy(void* c) { delete static_cast<RSWACache*>(c); }
int uocr_b200_cache_reset(void* c, int prefill_len) { return guarded([&] { static_cast<RSWACache*>(c)->reset(prefill_len); }); }
int uocr_b200_cache_write_prefill(void* c, int layer, const float* k, const float* v, int seq) {
    return guarded([&] { static_cast<RSWACache*>(c)->write_prefill(layer, k, v, seq); });
}
int uocr_b200_cache_append_decode(void* c, int layer, const float* k, const float* v) {
    return guarded([&] { static_cast<RSWACache*>(c)->append_decode(layer, k, v); });
}
int uocr_b200_cache_attention(const void* c, int layer, const float* q, int seq, int q_start, float* out, int heads, int causal) {
    return guarded([&] { static_cast<const RSWACache*>(c)->attention(layer, q, seq, q_start, out, heads, causal != 0); });
}
int uocr_b200_cache_len(const void* c, int l) { return static_cast<const RSWACache*>(c)->len(l); }
int uocr_b200_cache_ring_pos(const void* c, int l) { return static_cast<const RSWACache*>(c)->ring_pos(l); }
int uocr_b200_cache_ring_started(const void* c, int l) { return static_cast<const RSWACache*>(c)->ring_started(l) ? 1 : 0; }
int uocr_b200_cache_capacity(const void* c) { return static_cast<const RSWACache*>(c)->capacity(); }
int uocr_b200_cache_prefill_len(const void* c) { return static_cast<const RSWACache*>(c)->prefill_len(); }
const float* uocr_b200_cache_keys(const void* c, int l) { return static_cast<const RSWACache*>(c)->keys(l); }
const float* uocr_b200_cache_values(const void* c, int l) { return static_cast<const RSWACache*>(c)->values(l); }
size_t uocr_b200_cache_bytes(const void* c) { return static_cast<const RSWACache*>(c)->bytes(); }

}  // extern "C"
