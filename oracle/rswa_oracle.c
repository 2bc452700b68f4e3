/*
 * TEST INFRASTRUCTURE ONLY -- see rswa_oracle.h.  Plain-C restatement of the reference's CPU code
 * for the R-SWA KV-cache path.  Nothing here is shipped or called by the CUDA library.
 */
#include "rswa_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* =============================================================================================
 * bf16 helpers -- include/uocr/common.h:49-64 (widen = shift left 16; narrow = add 0x7fff + lsb,
 * shift right 16: round-to-nearest-even on the raw bits, NaN not special-cased).
 * ========================================================================================== */
uint16_t orc_f32_to_bf16(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    uint32_t odd = (u >> 16) & 1u;
    u += 0x7fffu + odd;
    return (uint16_t)(u >> 16);
}

float orc_bf16_to_f32(uint16_t h) {
    uint32_t u = (uint32_t)h << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

void orc_round_bf16_inplace(float* x, size_t n) {
    for (size_t i = 0; i < n; ++i) x[i] = orc_bf16_to_f32(orc_f32_to_bf16(x[i]));
}

/* =============================================================================================
 * R-SWA cache
 * ========================================================================================== */
struct orc_cache {
    int layers, kv_heads, head_dim, window;
    int prefill_len, capacity;
    float** k; /* per layer [capacity, kv_heads*head_dim] */
    float** v;
    int* len;
    int* ring_pos;
    unsigned char* ring_started;
};

/* configure(): src/scheduler/kv_cache.cpp:14-27 */
orc_cache* orc_cache_create(int layers, int kv_heads, int head_dim, int window) {
    orc_cache* c = (orc_cache*)calloc(1, sizeof(*c));
    c->layers = layers;
    c->kv_heads = kv_heads;
    c->head_dim = head_dim;
    c->window = window;
    c->k = (float**)calloc((size_t)layers, sizeof(float*));
    c->v = (float**)calloc((size_t)layers, sizeof(float*));
    c->len = (int*)calloc((size_t)layers, sizeof(int));
    c->ring_pos = (int*)calloc((size_t)layers, sizeof(int));
    c->ring_started = (unsigned char*)calloc((size_t)layers, 1);
    return c;
}

void orc_cache_destroy(orc_cache* c) {
    if (!c) return;
    for (int l = 0; l < c->layers; ++l) {
        free(c->k[l]);
        free(c->v[l]);
    }
    free(c->k);
    free(c->v);
    free(c->len);
    free(c->ring_pos);
    free(c->ring_started);
    free(c);
}

/* reset(P): src/scheduler/kv_cache.cpp:29-43 -- capacity = P + W, zero-filled K/V, len = P,
 * ring cursor cleared.  Negative P is the reference's UOCR_CHECK failure. */
int orc_cache_reset(orc_cache* c, int prefill_len) {
    if (prefill_len < 0) return -1;
    c->prefill_len = prefill_len;
    c->capacity = prefill_len + c->window;
    size_t n = (size_t)c->capacity * (size_t)c->kv_heads * (size_t)c->head_dim;
    for (int l = 0; l < c->layers; ++l) {
        free(c->k[l]);
        free(c->v[l]);
        c->k[l] = (float*)calloc(n ? n : 1, sizeof(float));
        c->v[l] = (float*)calloc(n ? n : 1, sizeof(float));
        c->len[l] = prefill_len;
        c->ring_pos[l] = 0;
        c->ring_started[l] = 0;
    }
    return 0;
}

/* write_prefill(): src/scheduler/kv_cache.cpp:45-52 -- rows [0,seq) <- k,v; len = prefill_len = seq
 * (capacity is deliberately NOT recomputed). */
int orc_cache_write_prefill(orc_cache* c, int layer, const float* k, const float* v, int seq) {
    if (seq > c->capacity) return -1;
    size_t row = (size_t)c->kv_heads * (size_t)c->head_dim;
    memcpy(c->k[layer], k, (size_t)seq * row * sizeof(float));
    memcpy(c->v[layer], v, (size_t)seq * row * sizeof(float));
    c->len[layer] = seq;
    c->prefill_len = seq;
    return 0;
}

/* append_decode(): src/scheduler/kv_cache.cpp:54-82 -- the ring state machine. */
void orc_cache_append_decode(orc_cache* c, int layer, const float* k, const float* v) {
    size_t row = (size_t)c->kv_heads * (size_t)c->head_dim;
    int n = c->len[layer];
    int full = c->prefill_len + c->window;
    int dst;
    if (n < full) { /* warm-up: linear growth */
        dst = n;
        c->len[layer] = n + 1;
        if (n + 1 >= full) {
            c->ring_started[layer] = 1;
            c->ring_pos[layer] = 0;
        }
    } else { /* steady state: overwrite slot P + ring_pos */
        if (!c->ring_started[layer]) {
            c->ring_started[layer] = 1;
            c->ring_pos[layer] = 0;
        }
        int rp = c->ring_pos[layer];
        dst = c->prefill_len + rp;
        c->ring_pos[layer] = (rp + 1) % c->window;
    }
    memcpy(c->k[layer] + (size_t)dst * row, k, row * sizeof(float));
    memcpy(c->v[layer] + (size_t)dst * row, v, row * sizeof(float));
}

/* attention(): src/scheduler/kv_cache.cpp:84-130 -- one key at a time, online softmax starting at
 * m = -inf, exp via libm, scale = 1/sqrt(head_dim), output acc/l (0 when nothing attended).  The
 * loop order and fp32 operation order are kept so results match the reference bit for bit when
 * compiled without fast-math. */
int orc_cache_attention(const orc_cache* c, int layer, const float* q, int seq, int q_start,
                        float* out, int heads, int causal) {
    int hd = c->head_dim;
    if (hd > 512) return -1;
    int kv_len = c->len[layer];
    int group = heads / c->kv_heads;
    float scale = 1.0f / sqrtf((float)hd);
    size_t row = (size_t)c->kv_heads * (size_t)hd;
    const float* kb = c->k[layer];
    const float* vb = c->v[layer];
    float acc[512];
    for (int s = 0; s < seq; ++s) {
        int qpos = q_start + s;
        int limit = kv_len;
        if (causal && qpos + 1 < limit) limit = qpos + 1;
        for (int h = 0; h < heads; ++h) {
            const float* qh = q + ((size_t)s * heads + h) * hd;
            int kvh = h / group;
            float m = -INFINITY, l = 0.0f;
            memset(acc, 0, sizeof(float) * (size_t)hd);
            for (int t = 0; t < limit; ++t) {
                const float* kt = kb + (size_t)t * row + (size_t)kvh * hd;
                const float* vt = vb + (size_t)t * row + (size_t)kvh * hd;
                float dot = 0.0f;
                for (int d = 0; d < hd; ++d) dot += qh[d] * kt[d];
                dot *= scale;
                float m_new = dot > m ? dot : m;
                float alpha = expf(m - m_new);
                float beta = expf(dot - m_new);
                l = l * alpha + beta;
                for (int d = 0; d < hd; ++d) acc[d] = acc[d] * alpha + beta * vt[d];
                m = m_new;
            }
            float inv = l > 0.0f ? 1.0f / l : 0.0f;
            float* oh = out + ((size_t)s * heads + h) * hd;
            for (int d = 0; d < hd; ++d) oh[d] = acc[d] * inv;
        }
    }
    return 0;
}

int orc_cache_len(const orc_cache* c, int layer) { return c->len[layer]; }
int orc_cache_ring_pos(const orc_cache* c, int layer) { return c->ring_pos[layer]; }
int orc_cache_ring_started(const orc_cache* c, int layer) { return c->ring_started[layer]; }
int orc_cache_capacity(const orc_cache* c) { return c->capacity; }
int orc_cache_prefill_len(const orc_cache* c) { return c->prefill_len; }
const float* orc_cache_keys(const orc_cache* c, int layer) { return c->k[layer]; }
const float* orc_cache_values(const orc_cache* c, int layer) { return c->v[layer]; }

/* bytes(): src/scheduler/kv_cache.cpp:132-137 */
size_t orc_cache_bytes(const orc_cache* c) {
    size_t n = (size_t)c->capacity * (size_t)c->kv_heads * (size_t)c->head_dim;
    return 2u * (size_t)c->layers * n * sizeof(float);
}

/* =============================================================================================
 * Offset arena with an offset-sorted, coalescing free list
 * ========================================================================================== */
typedef struct {
    size_t off, size;
} orc_span;

struct orc_pool {
    size_t total, used, peak, alignment;
    orc_span* fl; /* sorted by off */
    size_t n, cap;
};

static void fl_insert(orc_pool* p, size_t at, orc_span s) {
    if (p->n == p->cap) {
        p->cap = p->cap ? p->cap * 2 : 16;
        p->fl = (orc_span*)realloc(p->fl, p->cap * sizeof(orc_span));
    }
    memmove(p->fl + at + 1, p->fl + at, (p->n - at) * sizeof(orc_span));
    p->fl[at] = s;
    p->n++;
}

static void fl_erase(orc_pool* p, size_t at) {
    memmove(p->fl + at, p->fl + at + 1, (p->n - at - 1) * sizeof(orc_span));
    p->n--;
}

/* ctor + reserve(): src/scheduler/memory_pool.cpp:7-18 */
orc_pool* orc_pool_create(size_t bytes, size_t alignment) {
    orc_pool* p = (orc_pool*)calloc(1, sizeof(*p));
    p->alignment = alignment;
    if (bytes > 0) {
        p->total = bytes;
        orc_span all = {0, bytes};
        fl_insert(p, 0, all);
    }
    return p;
}

void orc_pool_destroy(orc_pool* p) {
    if (!p) return;
    free(p->fl);
    free(p);
}

/* reset(): src/scheduler/memory_pool.cpp:20-25 */
void orc_pool_reset(orc_pool* p) {
    p->used = p->peak = 0;
    p->n = 0;
    orc_span all = {0, p->total};
    fl_insert(p, 0, all);
}

/* allocate(): src/scheduler/memory_pool.cpp:27-52 -- first fit in offset order; the alignment pad
 * and the tail both go back on the list; `used` grows by pad + bytes; zero bytes -> offset 0. */
int64_t orc_pool_allocate(orc_pool* p, size_t bytes, size_t alignment) {
    if (bytes == 0) return 0;
    size_t a = alignment ? alignment : p->alignment;
    if (a == 0) a = 1;
    for (size_t i = 0; i < p->n; ++i) {
        size_t start = p->fl[i].off, size = p->fl[i].size;
        size_t pad = (a - start % a) % a;
        if (size < pad + bytes) continue;
        size_t off = start + pad;
        fl_erase(p, i);
        size_t at = i;
        if (pad > 0) {
            orc_span s = {start, pad};
            fl_insert(p, at++, s);
        }
        if (size > pad + bytes) {
            orc_span s = {off + bytes, size - pad - bytes};
            fl_insert(p, at, s);
        }
        p->used += pad + bytes;
        if (p->used > p->peak) p->peak = p->used;
        return (int64_t)off;
    }
    return -1;
}

/* free(): src/scheduler/memory_pool.cpp:54-74 -- sorted insert, `used -= bytes` only when it does
 * not underflow (the pad is never given back), merge with next, then previous with this. */
void orc_pool_free(orc_pool* p, int64_t offset, size_t bytes) {
    if (bytes == 0) return;
    size_t off = (size_t)offset;
    size_t at = 0;
    while (at < p->n && p->fl[at].off < off) ++at;
    orc_span s = {off, bytes};
    fl_insert(p, at, s);
    if (p->used >= bytes) p->used -= bytes;
    if (at + 1 < p->n && p->fl[at].off + p->fl[at].size == p->fl[at + 1].off) {
        p->fl[at].size += p->fl[at + 1].size;
        fl_erase(p, at + 1);
    }
    if (at > 0 && p->fl[at - 1].off + p->fl[at - 1].size == p->fl[at].off) {
        p->fl[at - 1].size += p->fl[at].size;
        fl_erase(p, at);
    }
}

size_t orc_pool_total(const orc_pool* p) { return p->total; }
size_t orc_pool_used(const orc_pool* p) { return p->used; }
size_t orc_pool_peak(const orc_pool* p) { return p->peak; }
size_t orc_pool_num_free_blocks(const orc_pool* p) { return p->n; }

/* fragmentation(): src/scheduler/memory_pool.cpp:76-85 */
double orc_pool_fragmentation(const orc_pool* p) {
    size_t sum = 0, big = 0;
    for (size_t i = 0; i < p->n; ++i) {
        sum += p->fl[i].size;
        if (p->fl[i].size > big) big = p->fl[i].size;
    }
    if (sum == 0) return 0.0;
    return 1.0 - (double)big / (double)sum;
}

/* =============================================================================================
 * Block manager: refcounted prefix arena + ring arena
 * ========================================================================================== */
typedef struct {
    char* key;
    int prefill_len;
    size_t bytes;
    int refcount;
    int64_t offset;
} orc_prefix;

struct orc_bm {
    orc_pool* prefix_pool;
    orc_pool* ring_pool;
    orc_prefix* e;
    size_t n, cap;
    size_t shared, peak_shared;
};

/* ctor: src/scheduler/block_manager.cpp:7-8 (both arenas use the default 256-byte alignment,
 * include/uocr/memory_pool.h:23) */
orc_bm* orc_bm_create(size_t prefix_pool_bytes, size_t ring_pool_bytes) {
    orc_bm* m = (orc_bm*)calloc(1, sizeof(*m));
    m->prefix_pool = orc_pool_create(prefix_pool_bytes, 256);
    m->ring_pool = orc_pool_create(ring_pool_bytes, 256);
    return m;
}

void orc_bm_destroy(orc_bm* m) {
    if (!m) return;
    for (size_t i = 0; i < m->n; ++i) free(m->e[i].key);
    free(m->e);
    orc_pool_destroy(m->prefix_pool);
    orc_pool_destroy(m->ring_pool);
    free(m);
}

/* recompute_shared(): src/scheduler/block_manager.cpp:46-52 */
static void bm_recount(orc_bm* m) {
    size_t s = 0;
    for (size_t i = 0; i < m->n; ++i)
        if (m->e[i].refcount >= 2) s += m->e[i].bytes;
    m->shared = s;
    if (s > m->peak_shared) m->peak_shared = s;
}

static long bm_find(const orc_bm* m, const char* key) {
    for (size_t i = 0; i < m->n; ++i)
        if (strcmp(m->e[i].key, key) == 0) return (long)i;
    return -1;
}

/* acquire_prefix(): src/scheduler/block_manager.cpp:10-32 */
int64_t orc_bm_acquire_prefix(orc_bm* m, const char* key, int prefill_len, size_t bytes,
                              int* refcount) {
    long i = bm_find(m, key);
    if (i >= 0) {
        m->e[i].refcount += 1;
        bm_recount(m);
        if (refcount) *refcount = m->e[i].refcount;
        return m->e[i].offset;
    }
    int64_t off = orc_pool_allocate(m->prefix_pool, bytes, 0);
    if (off < 0) return -1; /* "prefix pool exhausted" */
    if (m->n == m->cap) {
        m->cap = m->cap ? m->cap * 2 : 8;
        m->e = (orc_prefix*)realloc(m->e, m->cap * sizeof(orc_prefix));
    }
    orc_prefix* e = &m->e[m->n++];
    e->key = strdup(key);
    e->prefill_len = prefill_len;
    e->bytes = bytes;
    e->refcount = 1;
    e->offset = off;
    bm_recount(m);
    if (refcount) *refcount = 1;
    return off;
}

/* release_prefix(): src/scheduler/block_manager.cpp:34-44 -- unknown key is a no-op. */
void orc_bm_release_prefix(orc_bm* m, const char* key) {
    long i = bm_find(m, key);
    if (i < 0) return;
    m->e[i].refcount -= 1;
    if (m->e[i].refcount <= 0) {
        orc_pool_free(m->prefix_pool, m->e[i].offset, m->e[i].bytes);
        free(m->e[i].key);
        m->e[i] = m->e[m->n - 1];
        m->n--;
    }
    bm_recount(m);
}

/* allocate_ring / free_ring: src/scheduler/block_manager.cpp:54-56 */
int64_t orc_bm_allocate_ring(orc_bm* m, size_t bytes) {
    return orc_pool_allocate(m->ring_pool, bytes, 0);
}
void orc_bm_free_ring(orc_bm* m, int64_t offset, size_t bytes) {
    orc_pool_free(m->ring_pool, offset, bytes);
}

uint64_t orc_bm_live_prefixes(const orc_bm* m) { return m->n; }
uint64_t orc_bm_total_prefix_bytes(const orc_bm* m) {
    uint64_t t = 0;
    for (size_t i = 0; i < m->n; ++i) t += m->e[i].bytes;
    return t;
}
uint64_t orc_bm_shared_prefix_bytes(const orc_bm* m) { return m->shared; }
uint64_t orc_bm_peak_prefix_bytes(const orc_bm* m) { return m->peak_shared; }

/* stats(): src/scheduler/block_manager.cpp:66-77 */
void orc_bm_get_stats(const orc_bm* m, orc_bm_stats* o) {
    o->prefix_live_bytes = orc_pool_used(m->prefix_pool);
    o->prefix_peak_bytes = orc_pool_peak(m->prefix_pool);
    o->prefix_shared_bytes = m->shared;
    o->ring_live_bytes = orc_pool_used(m->ring_pool);
    o->ring_peak_bytes = orc_pool_peak(m->ring_pool);
    o->prefix_fragmentation = orc_pool_fragmentation(m->prefix_pool);
    o->ring_fragmentation = orc_pool_fragmentation(m->ring_pool);
    o->live_prefixes = m->n;
}

/* =============================================================================================
 * Continuous-batching scheduler
 * ========================================================================================== */
enum { ST_WAITING = 0, ST_PREFILLING = 1, ST_DECODING = 2, ST_FINISHED = 3 };

typedef struct {
    int state, prompt_len, n_out, max_new;
} orc_req;

struct orc_sched {
    int max_batch, min_batch;
    orc_req* r; /* ids are dense, handed out from 0: continuous_batch.cpp:10-19 */
    int n, cap;
    int* waiting;
    int w_head, w_tail, w_cap;
    int* running;
    int n_running, run_cap;
};

orc_sched* orc_sched_create(int max_batch_size, int min_batch_size) {
    orc_sched* s = (orc_sched*)calloc(1, sizeof(*s));
    s->max_batch = max_batch_size;
    s->min_batch = min_batch_size;
    return s;
}

void orc_sched_destroy(orc_sched* s) {
    if (!s) return;
    free(s->r);
    free(s->waiting);
    free(s->running);
    free(s);
}

/* add_request(): src/scheduler/continuous_batch.cpp:10-19 */
int orc_sched_add_request(orc_sched* s, int prompt_len, int max_new_tokens) {
    if (s->n == s->cap) {
        s->cap = s->cap ? s->cap * 2 : 16;
        s->r = (orc_req*)realloc(s->r, (size_t)s->cap * sizeof(orc_req));
    }
    if (s->w_tail == s->w_cap) {
        s->w_cap = s->w_cap ? s->w_cap * 2 : 16;
        s->waiting = (int*)realloc(s->waiting, (size_t)s->w_cap * sizeof(int));
    }
    int id = s->n++;
    s->r[id].state = ST_WAITING;
    s->r[id].prompt_len = prompt_len;
    s->r[id].n_out = 0;
    s->r[id].max_new = max_new_tokens;
    s->waiting[s->w_tail++] = id;
    return id;
}

static void run_push(orc_sched* s, int id) {
    if (s->n_running == s->run_cap) {
        s->run_cap = s->run_cap ? s->run_cap * 2 : 16;
        s->running = (int*)realloc(s->running, (size_t)s->run_cap * sizeof(int));
    }
    s->running[s->n_running++] = id;
}

/* build_batch(): src/scheduler/continuous_batch.cpp:21-57 -- running requests first (stop at
 * max_batch_size), then admit from the FIFO, then drop finished ids from the running set. */
void orc_sched_build_batch(orc_sched* s, int* prefill_ids, int* n_prefill, int* decode_ids,
                           int* n_decode, int cap) {
    int np = 0, nd = 0;
    for (int i = 0; i < s->n_running; ++i) {
        int id = s->running[i];
        if (s->r[id].state == ST_FINISHED) continue;
        if (np + nd >= s->max_batch) break;
        if (s->r[id].state == ST_DECODING && nd < cap) decode_ids[nd++] = id;
        else if (s->r[id].state == ST_PREFILLING && np < cap) prefill_ids[np++] = id;
    }
    while (s->w_head < s->w_tail && np + nd < s->max_batch) {
        int id = s->waiting[s->w_head++];
        s->r[id].state = ST_PREFILLING;
        run_push(s, id);
        if (np < cap) prefill_ids[np++] = id;
    }
    int keep = 0;
    for (int i = 0; i < s->n_running; ++i)
        if (s->r[s->running[i]].state != ST_FINISHED) s->running[keep++] = s->running[i];
    s->n_running = keep;
    *n_prefill = np;
    *n_decode = nd;
}

/* mark_prefilling / mark_prefilled: src/scheduler/continuous_batch.cpp:59-69 */
void orc_sched_mark_prefilling(orc_sched* s, int id) {
    if (id >= 0 && id < s->n) s->r[id].state = ST_PREFILLING;
}
void orc_sched_mark_prefilled(orc_sched* s, int id) {
    if (id >= 0 && id < s->n) s->r[id].state = ST_DECODING;
}

/* finish(): src/scheduler/continuous_batch.cpp:89-96 */
void orc_sched_finish(orc_sched* s, int id) {
    if (id < 0 || id >= s->n) return;
    s->r[id].state = ST_FINISHED;
    int keep = 0;
    for (int i = 0; i < s->n_running; ++i)
        if (s->running[i] != id) s->running[keep++] = s->running[i];
    s->n_running = keep;
}

/* add_token(): src/scheduler/continuous_batch.cpp:71-87 -- unknown id reports "finished". */
int orc_sched_add_token(orc_sched* s, int id, int token) {
    (void)token;
    if (id < 0 || id >= s->n) return 1;
    s->r[id].n_out += 1;
    if (s->r[id].n_out >= s->r[id].max_new) {
        orc_sched_finish(s, id);
        return 1;
    }
    return 0;
}

int orc_sched_state(const orc_sched* s, int id) {
    return (id >= 0 && id < s->n) ? s->r[id].state : -1;
}
int orc_sched_num_outputs(const orc_sched* s, int id) {
    return (id >= 0 && id < s->n) ? s->r[id].n_out : -1;
}
int orc_sched_has_work(const orc_sched* s) { return s->w_head < s->w_tail || s->n_running > 0; }
int orc_sched_running(const orc_sched* s, int* ids, int cap) {
    int n = s->n_running < cap ? s->n_running : cap;
    for (int i = 0; i < n; ++i) ids[i] = s->running[i];
    return s->n_running;
}

/* stats(): src/scheduler/continuous_batch.cpp:107-117 */
void orc_sched_get_stats(const orc_sched* s, orc_sched_stats* o) {
    memset(o, 0, sizeof(*o));
    for (int i = 0; i < s->n; ++i) {
        o->total_requests += 1;
        if (s->r[i].state == ST_FINISHED) {
            o->finished_requests += 1;
            o->prefill_tokens += (uint64_t)s->r[i].prompt_len;
            o->decode_tokens += (uint64_t)s->r[i].n_out;
        }
    }
    o->waiting = (uint64_t)(s->w_tail - s->w_head);
    o->running = (uint64_t)s->n_running;
    o->last_batch_size = (double)s->n_running;
}

/* =============================================================================================
 * Timed decode leg (CPU baseline of the benchmark)
 * ========================================================================================== */
static inline uint64_t mix64(uint64_t x) { /* splitmix64 finaliser */
    x += 0x9e3779b97f4a7c15ull;
    x = (x ^ (x >> 30)) * 0xbf58476d1ce4e5b9ull;
    x = (x ^ (x >> 27)) * 0x94d049bb133111ebull;
    return x ^ (x >> 31);
}

/* counter-based N(0,1): two hashed uniforms -> Box-Muller, then bf16-rounded so the fp32 cache holds
 * exactly what a bf16 cache would */
static void fill_normal_bf16(float* dst, size_t n, uint64_t seed, uint64_t stream) {
    for (size_t i = 0; i < n; i += 2) {
        uint64_t a = mix64(seed ^ mix64(stream * 0x100000001b3ull + i));
        uint64_t b = mix64(a);
        double u1 = ((double)(a >> 11) + 1.0) / 9007199254740993.0;
        double u2 = (double)(b >> 11) / 9007199254740992.0;
        double r = sqrt(-2.0 * log(u1));
        dst[i] = orc_bf16_to_f32(orc_f32_to_bf16((float)(r * cos(6.283185307179586 * u2))));
        if (i + 1 < n)
            dst[i + 1] = orc_bf16_to_f32(orc_f32_to_bf16((float)(r * sin(6.283185307179586 * u2))));
    }
}

static double now_s(void) {
    struct timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return (double)ts.tv_sec + 1e-9 * (double)ts.tv_nsec;
}

double orc_decode_bench(int n_seq, int layers, int kv_heads, int head_dim, int window,
                        const int* prefix_len, const int* pos, int steps, int threads,
                        uint64_t seed, double* checksum, int* threads_used) {
    size_t row = (size_t)kv_heads * (size_t)head_dim;
    int heads = kv_heads;
    orc_cache** caches = (orc_cache**)calloc((size_t)n_seq, sizeof(orc_cache*));
    int nthreads = 1;
#ifdef _OPENMP
    if (threads > 0) omp_set_num_threads(threads);
    nthreads = omp_get_max_threads();
#else
    (void)threads;
#endif
    if (threads_used) *threads_used = nthreads;

    /* state set-up (untimed): prefix, then pos[i] appends; only the last `window` rows survive, so
     * earlier appends reuse one scratch row */
#pragma omp parallel for schedule(dynamic)
    for (int i = 0; i < n_seq; ++i) {
        orc_cache* c = orc_cache_create(layers, kv_heads, head_dim, window);
        orc_cache_reset(c, prefix_len[i]);
        float* pk = (float*)malloc((size_t)(prefix_len[i] > 0 ? prefix_len[i] : 1) * row * sizeof(float));
        float* kr = (float*)malloc(row * sizeof(float));
        for (int l = 0; l < layers; ++l) {
            fill_normal_bf16(pk, (size_t)prefix_len[i] * row, seed, (uint64_t)(i * 64 + l) * 4 + 0);
            orc_cache_write_prefill(c, l, pk, pk, prefix_len[i]);
            for (int t = 0; t < pos[i]; ++t) {
                if (t == 0 || t >= pos[i] - window)
                    fill_normal_bf16(kr, row, seed, ((uint64_t)(i * 64 + l) * 4 + 1) * 1000003ull + (uint64_t)t);
                orc_cache_append_decode(c, l, kr, kr);
            }
        }
        free(pk);
        free(kr);
        caches[i] = c;
    }

    float* q = (float*)malloc((size_t)n_seq * layers * row * sizeof(float));
    float* kv = (float*)malloc((size_t)n_seq * layers * row * sizeof(float));
    float* out = (float*)malloc((size_t)n_seq * layers * (size_t)heads * head_dim * sizeof(float));
    fill_normal_bf16(q, (size_t)n_seq * layers * row, seed, 0xabcdefull);
    fill_normal_bf16(kv, (size_t)n_seq * layers * row, seed, 0x123457ull);

    double t0 = now_s();
    for (int st = 0; st < steps; ++st) {
#pragma omp parallel for schedule(dynamic) collapse(2)
        for (int i = 0; i < n_seq; ++i)
            for (int l = 0; l < layers; ++l) {
                size_t o = ((size_t)i * layers + l) * row;
                orc_cache_append_decode(caches[i], l, kv + o, kv + o);
                orc_cache_attention(caches[i], l, q + o, 1, orc_cache_len(caches[i], l) - 1, out + o,
                                    heads, 0);
            }
    }
    double dt = now_s() - t0;

    double cs = 0.0;
    for (size_t i = 0; i < (size_t)n_seq * layers * row; ++i) cs += (double)out[i];
    if (checksum) *checksum = cs;
    for (int i = 0; i < n_seq; ++i) orc_cache_destroy(caches[i]);
    free(caches);
    free(q);
    free(kv);
    free(out);
    return dt;
}

/* ---- RoPE: src/kernels/cpu_ops.cpp:146-180 (rope_row + rope) ------------------------------------
 * Same float arithmetic as the reference: powf / cosf / sinf on floats, the angle as an fp32 product
 * of the integer position and the frequency. */
void orc_rope(float* q, float* k, const int* positions, int seq, int n_heads, int n_kv_heads, int head_dim,
              float theta) {
    const int half = head_dim / 2;
    float* c = (float*)malloc(sizeof(float) * (size_t)(half > 0 ? half : 1));
    float* s = (float*)malloc(sizeof(float) * (size_t)(half > 0 ? half : 1));
    for (int t = 0; t < seq; ++t) {
        const int p = positions ? positions[t] : t;
        for (int i = 0; i < half; ++i) {
            const float freq = powf(theta, -2.0f * i / (float)head_dim);
            const float angle = p * freq;
            c[i] = cosf(angle);
            s[i] = sinf(angle);
        }
        for (int pass = 0; pass < 2; ++pass) {
            float* base = pass == 0 ? q : k;
            const int heads = pass == 0 ? n_heads : n_kv_heads;
            if (!base) continue;
            for (int h = 0; h < heads; ++h) {
                float* v = base + ((size_t)t * heads + h) * head_dim;
                for (int i = 0; i < half; ++i) {
                    const float x0 = v[i], x1 = v[i + half];
                    v[i] = x0 * c[i] - x1 * s[i];
                    v[i + half] = x0 * s[i] + x1 * c[i];
                }
            }
        }
    }
    free(c);
    free(s);
}
