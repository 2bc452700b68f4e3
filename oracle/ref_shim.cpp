// TEST INFRASTRUCTURE ONLY.  C shim over the UNMODIFIED reference classes, compiled together with
// the reference's own sources (taken from where the reference checkout lies, never copied) into
// oracle/_ref/libuocr_ref.so by oracle/Makefile.  It exports the same function set as
// rswa_oracle.h with the prefix `ref_` so one Python driver can run the restatement and the real
// reference side by side.  Used to pin the restatement, to generate tests/golden/, and as the
// "reference" CPU baseline of the benchmark.
#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <memory>
#include <string>
#include <vector>
#ifdef _OPENMP
#include <omp.h>
#endif

#include "uocr/block_manager.h"
#include "uocr/common.h"
#include "uocr/continuous_batch.h"
#include "uocr/kv_cache.h"
#include "uocr/memory_pool.h"
#include "uocr/ops.h"

#define REF_API extern "C" __attribute__((visibility("default")))

using namespace uocr;

// ---- bf16 -------------------------------------------------------------------------------------
REF_API uint16_t ref_f32_to_bf16(float f) { return f32_to_bf16(f); }
REF_API float ref_bf16_to_f32(uint16_t h) { return bf16_to_f32(h); }
REF_API void ref_round_bf16_inplace(float* x, size_t n) {
    for (size_t i = 0; i < n; ++i) x[i] = bf16_to_f32(f32_to_bf16(x[i]));
}

// ---- RoPE (src/kernels/cpu_ops.cpp) --------------------------------------------------------------
REF_API void ref_rope(float* q, float* k, const int* positions, int seq, int n_heads, int n_kv_heads, int head_dim,
                      float theta) {
    ops::rope(q, k, positions, seq, n_heads, n_kv_heads, head_dim, theta);
}

// ---- RSWACache ---------------------------------------------------------------------------------
REF_API void* ref_cache_create(int layers, int kv_heads, int head_dim, int window) {
    return new RSWACache(layers, kv_heads, head_dim, window);
}
REF_API void ref_cache_destroy(void* c) { delete static_cast<RSWACache*>(c); }
REF_API int ref_cache_reset(void* c, int prefill_len) {
    try {
        static_cast<RSWACache*>(c)->reset(prefill_len);
    } catch (const Error&) {
        return -1;
    }
    return 0;
}
REF_API int ref_cache_write_prefill(void* c, int layer, const float* k, const float* v, int seq) {
    try {
        static_cast<RSWACache*>(c)->write_prefill(layer, k, v, seq);
    } catch (const Error&) {
        return -1;
    }
    return 0;
}
REF_API void ref_cache_append_decode(void* c, int layer, const float* k, const float* v) {
    static_cast<RSWACache*>(c)->append_decode(layer, k, v);
}
REF_API int ref_cache_attention(const void* c, int layer, const float* q, int seq, int q_start,
                                float* out, int heads, int causal) {
    try {
        static_cast<const RSWACache*>(c)->attention(layer, q, seq, q_start, out, heads, causal != 0);
    } catch (const Error&) {
        return -1;
    }
    return 0;
}
REF_API int ref_cache_len(const void* c, int l) { return static_cast<const RSWACache*>(c)->len(l); }
REF_API int ref_cache_ring_pos(const void* c, int l) { return static_cast<const RSWACache*>(c)->ring_pos(l); }
REF_API int ref_cache_ring_started(const void* c, int l) { return static_cast<const RSWACache*>(c)->ring_started(l) ? 1 : 0; }
REF_API int ref_cache_capacity(const void* c) { return static_cast<const RSWACache*>(c)->capacity(); }
REF_API int ref_cache_prefill_len(const void* c) { return static_cast<const RSWACache*>(c)->prefill_len(); }
REF_API const float* ref_cache_keys(const void* c, int l) { return static_cast<const RSWACache*>(c)->keys(l); }
REF_API const float* ref_cache_values(const void* c, int l) { return static_cast<const RSWACache*>(c)->values(l); }
REF_API size_t ref_cache_bytes(const void* c) { return static_cast<const RSWACache*>(c)->bytes(); }

// ---- MemoryPool --------------------------------------------------------------------------------
REF_API void* ref_pool_create(size_t bytes, size_t alignment) { return new MemoryPool(bytes, alignment); }
REF_API void ref_pool_destroy(void* p) { delete static_cast<MemoryPool*>(p); }
REF_API void ref_pool_reset(void* p) { static_cast<MemoryPool*>(p)->reset(); }
REF_API int64_t ref_pool_allocate(void* p, size_t bytes, size_t alignment) {
    return static_cast<MemoryPool*>(p)->allocate(bytes, alignment);
}
REF_API void ref_pool_free(void* p, int64_t off, size_t bytes) { static_cast<MemoryPool*>(p)->free(off, bytes); }
REF_API size_t ref_pool_total(const void* p) { return static_cast<const MemoryPool*>(p)->total(); }
REF_API size_t ref_pool_used(const void* p) { return static_cast<const MemoryPool*>(p)->used(); }
REF_API size_t ref_pool_peak(const void* p) { return static_cast<const MemoryPool*>(p)->peak(); }
REF_API size_t ref_pool_num_free_blocks(const void* p) { return static_cast<const MemoryPool*>(p)->num_free_blocks(); }
REF_API double ref_pool_fragmentation(const void* p) { return static_cast<const MemoryPool*>(p)->fragmentation(); }

// ---- BlockManager ------------------------------------------------------------------------------
struct ref_bm_stats {
    uint64_t prefix_live_bytes, prefix_peak_bytes, prefix_shared_bytes;
    uint64_t ring_live_bytes, ring_peak_bytes;
    double prefix_fragmentation, ring_fragmentation;
    uint64_t live_prefixes;
};
REF_API void* ref_bm_create(size_t prefix_bytes, size_t ring_bytes) { return new BlockManager(prefix_bytes, ring_bytes); }
REF_API void ref_bm_destroy(void* m) { delete static_cast<BlockManager*>(m); }
REF_API int64_t ref_bm_acquire_prefix(void* m, const char* key, int prefill_len, size_t bytes, int* refcount) {
    try {
        PrefixEntry* e = static_cast<BlockManager*>(m)->acquire_prefix(key, prefill_len, bytes);
        if (refcount) *refcount = e->refcount;
        return e->offset;
    } catch (const Error&) {
        return -1;
    }
}
REF_API void ref_bm_release_prefix(void* m, const char* key) { static_cast<BlockManager*>(m)->release_prefix(key); }
REF_API int64_t ref_bm_allocate_ring(void* m, size_t bytes) { return static_cast<BlockManager*>(m)->allocate_ring(bytes); }
REF_API void ref_bm_free_ring(void* m, int64_t off, size_t bytes) { static_cast<BlockManager*>(m)->free_ring(off, bytes); }
REF_API uint64_t ref_bm_live_prefixes(const void* m) { return static_cast<const BlockManager*>(m)->live_prefixes(); }
REF_API uint64_t ref_bm_total_prefix_bytes(const void* m) { return static_cast<const BlockManager*>(m)->total_prefix_bytes(); }
REF_API uint64_t ref_bm_shared_prefix_bytes(const void* m) { return static_cast<const BlockManager*>(m)->shared_prefix_bytes(); }
REF_API uint64_t ref_bm_peak_prefix_bytes(const void* m) { return static_cast<const BlockManager*>(m)->peak_prefix_bytes(); }
REF_API void ref_bm_get_stats(const void* m, ref_bm_stats* o) {
    BlockManager::Stats s = static_cast<const BlockManager*>(m)->stats();
    o->prefix_live_bytes = s.prefix_live_bytes;
    o->prefix_peak_bytes = s.prefix_peak_bytes;
    o->prefix_shared_bytes = s.prefix_shared_bytes;
    o->ring_live_bytes = s.ring_live_bytes;
    o->ring_peak_bytes = s.ring_peak_bytes;
    o->prefix_fragmentation = s.prefix_fragmentation;
    o->ring_fragmentation = s.ring_fragmentation;
    o->live_prefixes = s.live_prefixes;
}

// ---- ContinuousBatchScheduler ------------------------------------------------------------------
struct ref_sched_stats {
    uint64_t total_requests, finished_requests, prefill_tokens, decode_tokens;
    uint64_t waiting, running;
    double last_batch_size;
};
REF_API void* ref_sched_create(int max_batch, int min_batch) { return new ContinuousBatchScheduler(max_batch, min_batch); }
REF_API void ref_sched_destroy(void* s) { delete static_cast<ContinuousBatchScheduler*>(s); }
REF_API int ref_sched_add_request(void* s, int prompt_len, int max_new_tokens) {
    Request r;
    r.prompt_tokens.assign(static_cast<size_t>(prompt_len), 1);
    r.max_new_tokens = max_new_tokens;
    return static_cast<ContinuousBatchScheduler*>(s)->add_request(std::move(r));
}
REF_API void ref_sched_build_batch(void* s, int* prefill_ids, int* n_prefill, int* decode_ids, int* n_decode, int cap) {
    Batch b = static_cast<ContinuousBatchScheduler*>(s)->build_batch();
    int np = 0, nd = 0;
    for (int id : b.prefill) if (np < cap) prefill_ids[np++] = id;
    for (int id : b.decode) if (nd < cap) decode_ids[nd++] = id;
    *n_prefill = np;
    *n_decode = nd;
}
REF_API void ref_sched_mark_prefilled(void* s, int id) { static_cast<ContinuousBatchScheduler*>(s)->mark_prefilled(id); }
REF_API void ref_sched_mark_prefilling(void* s, int id) { static_cast<ContinuousBatchScheduler*>(s)->mark_prefilling(id); }
REF_API int ref_sched_add_token(void* s, int id, int token) { return static_cast<ContinuousBatchScheduler*>(s)->add_token(id, token) ? 1 : 0; }
REF_API void ref_sched_finish(void* s, int id) { static_cast<ContinuousBatchScheduler*>(s)->finish(id); }
REF_API int ref_sched_state(const void* s, int id) {
    const Request* r = static_cast<const ContinuousBatchScheduler*>(s)->get(id);
    return r ? static_cast<int>(r->state) : -1;
}
REF_API int ref_sched_num_outputs(const void* s, int id) {
    const Request* r = static_cast<const ContinuousBatchScheduler*>(s)->get(id);
    return r ? static_cast<int>(r->output_tokens.size()) : -1;
}
REF_API int ref_sched_has_work(const void* s) { return static_cast<const ContinuousBatchScheduler*>(s)->has_work() ? 1 : 0; }
REF_API int ref_sched_running(const void* s, int* ids, int cap) {
    const std::vector<int>& r = static_cast<const ContinuousBatchScheduler*>(s)->running();
    for (size_t i = 0; i < r.size() && static_cast<int>(i) < cap; ++i) ids[i] = r[i];
    return static_cast<int>(r.size());
}
REF_API void ref_sched_get_stats(const void* s, ref_sched_stats* o) {
    auto st = static_cast<const ContinuousBatchScheduler*>(s)->stats();
    o->total_requests = st.total_requests;
    o->finished_requests = st.finished_requests;
    o->prefill_tokens = st.prefill_tokens;
    o->decode_tokens = st.decode_tokens;
    o->waiting = st.waiting;
    o->running = st.running;
    o->last_batch_size = st.last_batch_size;
}

// ---- timed decode leg: OpenMP lives in this harness, around unmodified RSWACache calls ----------
static inline uint64_t mix64(uint64_t x) {
    x += 0x9e3779b97f4a7c15ull;
    x = (x ^ (x >> 30)) * 0xbf58476d1ce4e5b9ull;
    x = (x ^ (x >> 27)) * 0x94d049bb133111ebull;
    return x ^ (x >> 31);
}
static void fill_normal_bf16(float* dst, size_t n, uint64_t seed, uint64_t stream) {
    for (size_t i = 0; i < n; i += 2) {
        uint64_t a = mix64(seed ^ mix64(stream * 0x100000001b3ull + i));
        uint64_t b = mix64(a);
        double u1 = (static_cast<double>(a >> 11) + 1.0) / 9007199254740993.0;
        double u2 = static_cast<double>(b >> 11) / 9007199254740992.0;
        double r = std::sqrt(-2.0 * std::log(u1));
        dst[i] = bf16_to_f32(f32_to_bf16(static_cast<float>(r * std::cos(6.283185307179586 * u2))));
        if (i + 1 < n)
            dst[i + 1] = bf16_to_f32(f32_to_bf16(static_cast<float>(r * std::sin(6.283185307179586 * u2))));
    }
}

REF_API double ref_decode_bench(int n_seq, int layers, int kv_heads, int head_dim, int window,
                                const int* prefix_len, const int* pos, int steps, int threads,
                                uint64_t seed, double* checksum, int* threads_used) {
    const size_t row = static_cast<size_t>(kv_heads) * head_dim;
    const int heads = kv_heads;
    int nthreads = 1;
#ifdef _OPENMP
    if (threads > 0) omp_set_num_threads(threads);
    nthreads = omp_get_max_threads();
#endif
    if (threads_used) *threads_used = nthreads;
    std::vector<std::unique_ptr<RSWACache>> caches(static_cast<size_t>(n_seq));
#pragma omp parallel for schedule(dynamic)
    for (int i = 0; i < n_seq; ++i) {
        auto c = std::make_unique<RSWACache>(layers, kv_heads, head_dim, window);
        c->reset(prefix_len[i]);
        std::vector<float> pk(static_cast<size_t>(prefix_len[i]) * row), kr(row);
        for (int l = 0; l < layers; ++l) {
            fill_normal_bf16(pk.data(), pk.size(), seed, static_cast<uint64_t>(i * 64 + l) * 4 + 0);
            c->write_prefill(l, pk.data(), pk.data(), prefix_len[i]);
            for (int t = 0; t < pos[i]; ++t) {
                if (t == 0 || t >= pos[i] - window)
                    fill_normal_bf16(kr.data(), row, seed,
                                     (static_cast<uint64_t>(i * 64 + l) * 4 + 1) * 1000003ull + static_cast<uint64_t>(t));
                c->append_decode(l, kr.data(), kr.data());
            }
        }
        caches[static_cast<size_t>(i)] = std::move(c);
    }
    const size_t n = static_cast<size_t>(n_seq) * layers * row;
    std::vector<float> q(n), kv(n), out(n);
    fill_normal_bf16(q.data(), n, seed, 0xabcdefull);
    fill_normal_bf16(kv.data(), n, seed, 0x123457ull);

    auto t0 = std::chrono::steady_clock::now();
    for (int st = 0; st < steps; ++st) {
#pragma omp parallel for schedule(dynamic) collapse(2)
        for (int i = 0; i < n_seq; ++i)
            for (int l = 0; l < layers; ++l) {
                const size_t o = (static_cast<size_t>(i) * layers + l) * row;
                RSWACache& c = *caches[static_cast<size_t>(i)];
                c.append_decode(l, kv.data() + o, kv.data() + o);
                c.attention(l, q.data() + o, 1, c.length(l) - 1, out.data() + o, heads, false);
            }
    }
    const double dt = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    double cs = 0.0;
    for (size_t i = 0; i < n; ++i) cs += static_cast<double>(out[i]);
    if (checksum) *checksum = cs;
    return dt;
}
