/*
 * TEST INFRASTRUCTURE ONLY -- CPU restatement of the Unlimited-OCR R-SWA KV-cache path.
 *
 * This is the checker the CUDA path is compared against.  It is never linked into, imported by or
 * called from the shipped library; only the test-suite, the smoke check and the CPU-baseline leg of
 * the benchmark may load it.
 *
 * Every function restates one piece of the reference engine in plain C and cites the reference
 * file:line it follows (paths are relative to the reference project root).  Parity of this
 * restatement is pinned two ways: against the compiled, unmodified reference sources (the optional
 * oracle/_ref/libuocr_ref.so built by oracle/Makefile) on seeded random traces, and against the
 * golden vectors committed under tests/golden/ that were produced by that compiled reference.
 */
#ifndef RSWA_ORACLE_H
#define RSWA_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- bf16 rounding: include/uocr/common.h:49-64 ------------------------------------------- */
uint16_t orc_f32_to_bf16(float f);
float orc_bf16_to_f32(uint16_t h);
void orc_round_bf16_inplace(float* x, size_t n); /* x <- widen(round_bf16(x)) */

/* ---- RoPE in place on q [seq][n_heads][hd] and k [seq][n_kv_heads][hd] (k may be null):
 * src/kernels/cpu_ops.cpp:157-180.  Half-split pairs (i, i + hd/2), freq = powf(theta, -2i/hd),
 * angle = position * freq in fp32, positions == null means 0..seq-1. */
void orc_rope(float* q, float* k, const int* positions, int seq, int n_heads, int n_kv_heads, int head_dim,
              float theta);

/* ---- R-SWA cache: include/uocr/kv_cache.h:23-86, src/scheduler/kv_cache.cpp:10-137 ---------- */
typedef struct orc_cache orc_cache;
orc_cache* orc_cache_create(int layers, int kv_heads, int head_dim, int window);
void orc_cache_destroy(orc_cache* c);
int orc_cache_reset(orc_cache* c, int prefill_len);               /* 0 ok, -1 = reference would throw */
int orc_cache_write_prefill(orc_cache* c, int layer, const float* k, const float* v, int seq);
void orc_cache_append_decode(orc_cache* c, int layer, const float* k, const float* v);
int orc_cache_attention(const orc_cache* c, int layer, const float* q, int seq, int q_start,
                        float* out, int heads, int causal);
int orc_cache_len(const orc_cache* c, int layer);
int orc_cache_ring_pos(const orc_cache* c, int layer);
int orc_cache_ring_started(const orc_cache* c, int layer);
int orc_cache_capacity(const orc_cache* c);
int orc_cache_prefill_len(const orc_cache* c);
const float* orc_cache_keys(const orc_cache* c, int layer);
const float* orc_cache_values(const orc_cache* c, int layer);
size_t orc_cache_bytes(const orc_cache* c);

/* ---- arena: include/uocr/memory_pool.h:16-51, src/scheduler/memory_pool.cpp:7-85 ------------ */
typedef struct orc_pool orc_pool;
orc_pool* orc_pool_create(size_t bytes, size_t alignment);
void orc_pool_destroy(orc_pool* p);
void orc_pool_reset(orc_pool* p);
int64_t orc_pool_allocate(orc_pool* p, size_t bytes, size_t alignment);
void orc_pool_free(orc_pool* p, int64_t offset, size_t bytes);
size_t orc_pool_total(const orc_pool* p);
size_t orc_pool_used(const orc_pool* p);
size_t orc_pool_peak(const orc_pool* p);
size_t orc_pool_num_free_blocks(const orc_pool* p);
double orc_pool_fragmentation(const orc_pool* p);

/* ---- block manager: include/uocr/block_manager.h:25-79, src/scheduler/block_manager.cpp ----- */
typedef struct orc_bm orc_bm;
typedef struct {
    uint64_t prefix_live_bytes, prefix_peak_bytes, prefix_shared_bytes;
    uint64_t ring_live_bytes, ring_peak_bytes;
    double prefix_fragmentation, ring_fragmentation;
    uint64_t live_prefixes;
} orc_bm_stats;
orc_bm* orc_bm_create(size_t prefix_pool_bytes, size_t ring_pool_bytes);
void orc_bm_destroy(orc_bm* m);
/* returns the arena offset of the entry (>=0) and its refcount, or -1 when the reference throws
 * "prefix pool exhausted" */
int64_t orc_bm_acquire_prefix(orc_bm* m, const char* key, int prefill_len, size_t bytes, int* refcount);
void orc_bm_release_prefix(orc_bm* m, const char* key);
int64_t orc_bm_allocate_ring(orc_bm* m, size_t bytes);
void orc_bm_free_ring(orc_bm* m, int64_t offset, size_t bytes);
uint64_t orc_bm_live_prefixes(const orc_bm* m);
uint64_t orc_bm_total_prefix_bytes(const orc_bm* m);
uint64_t orc_bm_shared_prefix_bytes(const orc_bm* m);
uint64_t orc_bm_peak_prefix_bytes(const orc_bm* m);
void orc_bm_get_stats(const orc_bm* m, orc_bm_stats* out);

/* ---- scheduler: include/uocr/continuous_batch.h:21-104, src/scheduler/continuous_batch.cpp -- */
typedef struct orc_sched orc_sched;
typedef struct {
    uint64_t total_requests, finished_requests, prefill_tokens, decode_tokens;
    uint64_t waiting, running;
    double last_batch_size;
} orc_sched_stats;
orc_sched* orc_sched_create(int max_batch_size, int min_batch_size);
void orc_sched_destroy(orc_sched* s);
int orc_sched_add_request(orc_sched* s, int prompt_len, int max_new_tokens);
/* fills prefill_ids / decode_ids (caller arrays of capacity cap); counts returned through n_* */
void orc_sched_build_batch(orc_sched* s, int* prefill_ids, int* n_prefill, int* decode_ids,
                           int* n_decode, int cap);
void orc_sched_mark_prefilled(orc_sched* s, int id);
void orc_sched_mark_prefilling(orc_sched* s, int id);
int orc_sched_add_token(orc_sched* s, int id, int token); /* 1 when finished */
void orc_sched_finish(orc_sched* s, int id);
int orc_sched_state(const orc_sched* s, int id);          /* 0 W,1 P,2 D,3 F, -1 unknown */
int orc_sched_num_outputs(const orc_sched* s, int id);
int orc_sched_has_work(const orc_sched* s);
int orc_sched_running(const orc_sched* s, int* ids, int cap);
void orc_sched_get_stats(const orc_sched* s, orc_sched_stats* out);

/* ---- timed decode leg for the benchmark's CPU baseline ------------------------------------- */
/* Runs `steps` decode steps (append + non-causal attention, every layer) over `n_seq` caches whose
 * state was reached by `pos[i]` appends after a prefix of `prefix_len[i]`; OpenMP over independent
 * (sequence, layer) units in the harness, as the reference's own attention has no threading
 * (src/scheduler/kv_cache.cpp:84-130).  Returns seconds spent in the timed decode loop. */
double orc_decode_bench(int n_seq, int layers, int kv_heads, int head_dim, int window,
                        const int* prefix_len, const int* pos, int steps, int threads,
                        uint64_t seed, double* checksum, int* threads_used);

#ifdef __cplusplus
}
#endif
#endif
