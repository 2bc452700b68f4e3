/*
 * C ABI over the host-side classes of the R-SWA path (same shared library).  For callers that bind
 * through an FFI instead of including the C++ headers, and for driving those classes from the test
 * suite with the same scripts that drive the CPU oracle.  Handles are opaque; every function that
 * can fail returns a negative value or an int status as noted.
 *
 * Mirrors, one function per method:
 *   uocr::MemoryPool                 include/uocr/memory_pool.h:16-51
 *   uocr::BlockManager               include/uocr/block_manager.h:25-79
 *   uocr::ContinuousBatchScheduler   include/uocr/continuous_batch.h:21-104
 *   uocr::RSWACache                  include/uocr/kv_cache.h:23-86   (device-backed)
 */
#ifndef UOCR_RSWA_B200_HOST_H
#define UOCR_RSWA_B200_HOST_H

#include "uocr_rswa_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

/* ---- MemoryPool -------------------------------------------------------------------------------- */
UOCR_B200_API void* uocr_b200_pool_create(size_t bytes, size_t alignment);
UOCR_B200_API void uocr_b200_pool_destroy(void* pool);
UOCR_B200_API void uocr_b200_pool_reset(void* pool);
UOCR_B200_API int64_t uocr_b200_pool_allocate(void* pool, size_t bytes, size_t alignment); /* -1: no fit */
UOCR_B200_API void uocr_b200_pool_free(void* pool, int64_t offset, size_t bytes);
UOCR_B200_API size_t uocr_b200_pool_total(const void* pool);
UOCR_B200_API size_t uocr_b200_pool_used(const void* pool);
UOCR_B200_API size_t uocr_b200_pool_peak(const void* pool);
UOCR_B200_API size_t uocr_b200_pool_num_free_blocks(const void* pool);
UOCR_B200_API double uocr_b200_pool_fragmentation(const void* pool);

/* ---- BlockManager ------------------------------------------------------------------------------- */
typedef struct {
    uint64_t prefix_live_bytes, prefix_peak_bytes, prefix_shared_bytes;
    uint64_t ring_live_bytes, ring_peak_bytes;
    double prefix_fragmentation, ring_fragmentation;
    uint64_t live_prefixes;
} uocr_b200_bm_stats;
UOCR_B200_API void* uocr_b200_bm_create(size_t prefix_pool_bytes, size_t ring_pool_bytes);
UOCR_B200_API void uocr_b200_bm_destroy(void* bm);
/* arena offset of the entry and its refcount; -1 when the prefix pool is exhausted (the C++ method throws) */
UOCR_B200_API int64_t uocr_b200_bm_acquire_prefix(void* bm, const char* key, int prefill_len, size_t bytes, int* refcount);
UOCR_B200_API void uocr_b200_bm_release_prefix(void* bm, const char* key);
UOCR_B200_API int64_t uocr_b200_bm_allocate_ring(void* bm, size_t bytes);
UOCR_B200_API void uocr_b200_bm_free_ring(void* bm, int64_t offset, size_t bytes);
UOCR_B200_API uint64_t uocr_b200_bm_live_prefixes(const void* bm);
UOCR_B200_API uint64_t uocr_b200_bm_total_prefix_bytes(const void* bm);
UOCR_B200_API uint64_t uocr_b200_bm_shared_prefix_bytes(const void* bm);
UOCR_B200_API uint64_t uocr_b200_bm_peak_prefix_bytes(const void* bm);
UOCR_B200_API void uocr_b200_bm_get_stats(const void* bm, uocr_b200_bm_stats* out);

/* ---- ContinuousBatchScheduler --------------------------------------------------------------------- */
typedef struct {
    uint64_t total_requests, finished_requests, prefill_tokens, decode_tokens;
    uint64_t waiting, running;
    double last_batch_size;
} uocr_b200_sched_stats;
UOCR_B200_API void* uocr_b200_sched_create(int max_batch_size, int min_batch_size);
UOCR_B200_API void uocr_b200_sched_destroy(void* s);
UOCR_B200_API int uocr_b200_sched_add_request(void* s, int prompt_len, int max_new_tokens);
UOCR_B200_API void uocr_b200_sched_build_batch(void* s, int* prefill_ids, int* n_prefill, int* decode_ids, int* n_decode, int cap);
UOCR_B200_API void uocr_b200_sched_mark_prefilled(void* s, int id);
UOCR_B200_API void uocr_b200_sched_mark_prefilling(void* s, int id);
UOCR_B200_API int uocr_b200_sched_add_token(void* s, int id, int token); /* 1 when the request finished */
UOCR_B200_API void uocr_b200_sched_finish(void* s, int id);
UOCR_B200_API int uocr_b200_sched_state(const void* s, int id);          /* 0 W, 1 P, 2 D, 3 F, -1 unknown */
UOCR_B200_API int uocr_b200_sched_num_outputs(const void* s, int id);
UOCR_B200_API int uocr_b200_sched_has_work(const void* s);
UOCR_B200_API int uocr_b200_sched_running(const void* s, int* ids, int cap);
UOCR_B200_API void uocr_b200_sched_get_stats(const void* s, uocr_b200_sched_stats* out);

/* ---- RSWACache (host pointers in and out; the KV lives on the current CUDA device) ---------------- */
UOCR_B200_API void* uocr_b200_cache_create(int layers, int kv_heads, int head_dim, int window);
UOCR_B200_API int uocr_b200_cache_set_kv_dtype(void* c, int dtype); /* UOCR_B200_F32 / UOCR_B200_BF16 */
UOCR_B200_API void uocr_b200_cache_destroy(void* c);
UOCR_B200_API int uocr_b200_cache_reset(void* c, int prefill_len);  /* 0 ok, -1 = uocr::Error (see last_error) */
UOCR_B200_API int uocr_b200_cache_write_prefill(void* c, int layer, const float* k, const float* v, int seq);
UOCR_B200_API int uocr_b200_cache_append_decode(void* c, int layer, const float* k, const float* v);
UOCR_B200_API int uocr_b200_cache_attention(const void* c, int layer, const float* q, int seq, int q_start, float* out, int heads, int causal);
UOCR_B200_API int uocr_b200_cache_len(const void* c, int layer);
UOCR_B200_API int uocr_b200_cache_ring_pos(const void* c, int layer);
UOCR_B200_API int uocr_b200_cache_ring_started(const void* c, int layer);
UOCR_B200_API int uocr_b200_cache_capacity(const void* c);
UOCR_B200_API int uocr_b200_cache_prefill_len(const void* c);
UOCR_B200_API const float* uocr_b200_cache_keys(const void* c, int layer);
UOCR_B200_API const float* uocr_b200_cache_values(const void* c, int layer);
UOCR_B200_API size_t uocr_b200_cache_bytes(const void* c);

#ifdef __cplusplus
}
#endif
#endif
