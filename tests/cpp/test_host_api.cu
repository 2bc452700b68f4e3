// GPU tests of the C++ host API (uocr::RSWACache, uocr::cuda::GpuRSWACache, the uocr::cuda::rswa_*
// free functions with the reference's signatures, uocr::cuda::PagedBatchKV, uocr::SlotAllocator)
// against the CPU oracle (oracle/rswa_oracle.h -- test infrastructure, linked here as the checker).
// Cache contents and cursors must be bit-equal; attention within 2e-5.
#include <cuda_runtime.h>

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "rswa_oracle.h"
#include "uocr/cuda_ops.h"
#include "uocr/gpu_cache.h"
#include "uocr/kv_cache.h"

using namespace uocr;

static int g_fail = 0;
#define EXPECT(cond)                                                          \
    do {                                                                      \
        if (!(cond)) {                                                        \
            std::printf("  FAIL %s:%d: %s\n", __FILE__, __LINE__, #cond);     \
            ++g_fail;                                                         \
        }                                                                     \
    } while (0)

static uint64_t g_state = 0x9e3779b97f4a7c15ull;
static float rnd() {  // sum of four uniforms, centred: cheap bell-shaped values, exactly representable
    float s = 0.f;
    for (int i = 0; i < 4; ++i) {
        g_state = g_state * 6364136223846793005ull + 1442695040888963407ull;
        s += static_cast<float>((g_state >> 40) & 0xffff) / 65536.0f;
    }
    return (s - 2.0f) * 1.7f;
}
static std::vector<float> rvec(size_t n) {
    std::vector<float> v(n);
    for (auto& x : v) x = rnd();
    return v;
}
template <typename T>
static T* dev(const std::vector<T>& h) {
    T* d = nullptr;
    cudaMalloc(&d, std::max<size_t>(h.size(), 1) * sizeof(T));
    cudaMemcpy(d, h.data(), h.size() * sizeof(T), cudaMemcpyHostToDevice);
    return d;
}
template <typename T>
static std::vector<T> host(const T* d, size_t n) {
    std::vector<T> h(n);
    cudaMemcpy(h.data(), d, n * sizeof(T), cudaMemcpyDeviceToHost);
    return h;
}
static float max_abs_diff(const std::vector<float>& a, const float* b) {
    float m = 0.f;
    for (size_t i = 0; i < a.size(); ++i) m = std::max(m, std::fabs(a[i] - b[i]));
    return m;
}

// ---- RSWACache (host pointers) -----------------------------------------------------------------------
static void test_rswa_cache_host_interface() {
    std::printf("RSWACache (device-backed, host interface)\n");
    const int L = 2, kvh = 2, hd = 16, W = 8, P = 5, heads = 4, row = kvh * hd;
    RSWACache c(L, kvh, hd, W);
    orc_cache* o = orc_cache_create(L, kvh, hd, W);
    c.reset(P);
    orc_cache_reset(o, P);
    EXPECT(c.capacity() == P + W && c.prefill_len() == P && c.length(0) == P);
    for (int l = 0; l < L; ++l) {
        auto k = rvec(P * row), v = rvec(P * row);
        c.write_prefill(l, k.data(), v.data(), P);
        orc_cache_write_prefill(o, l, k.data(), v.data(), P);
    }
    for (int t = 0; t < 3 * W + 1; ++t)
        for (int l = 0; l < L; ++l) {
            auto k = rvec(row), v = rvec(row);
            c.append_decode(l, k.data(), v.data());
            orc_cache_append_decode(o, l, k.data(), v.data());
            EXPECT(c.length(l) == orc_cache_len(o, l) && c.ring_pos(l) == orc_cache_ring_pos(o, l));
            EXPECT(c.ring_started(l) == (orc_cache_ring_started(o, l) != 0));
        }
    for (int l = 0; l < L; ++l) {
        const size_t n = static_cast<size_t>(c.capacity()) * row;
        EXPECT(std::memcmp(c.keys(l), orc_cache_keys(o, l), n * 4) == 0);
        EXPECT(std::memcmp(c.values(l), orc_cache_values(o, l), n * 4) == 0);
        auto q = rvec(heads * hd);
        std::vector<float> got(heads * hd, NAN), want(heads * hd);
        c.attention(l, q.data(), 1, c.length(l) - 1, got.data(), heads, false);
        orc_cache_attention(o, l, q.data(), 1, orc_cache_len(o, l) - 1, want.data(), heads, 0);
        EXPECT(max_abs_diff(got, want.data()) < 2e-5f);
    }
    // a write through mutable_keys() reaches the device before the next operation
    float* mk = c.mutable_keys(0);
    float* ok = const_cast<float*>(orc_cache_keys(o, 0));
    mk[3 * row + 1] = 7.5f;
    ok[3 * row + 1] = 7.5f;
    auto q = rvec(heads * hd);
    std::vector<float> got(heads * hd, NAN), want(heads * hd);
    c.attention(0, q.data(), 1, c.length(0) - 1, got.data(), heads, false);
    orc_cache_attention(o, 0, q.data(), 1, orc_cache_len(o, 0) - 1, want.data(), heads, 0);
    EXPECT(max_abs_diff(got, want.data()) < 2e-5f);
    EXPECT(c.keys(0)[3 * row + 1] == 7.5f);
    EXPECT(c.bytes() == orc_cache_bytes(o));
    bool threw = false;
    try {
        c.write_prefill(0, q.data(), q.data(), c.capacity() + 1);
    } catch (const Error&) {
        threw = true;
    }
    EXPECT(threw);
    orc_cache_destroy(o);
}

// ---- GpuRSWACache (device pointers) ----------------------------------------------------------------------
static void test_gpu_cache_device_interface() {
    std::printf("cuda::GpuRSWACache\n");
    const int L = 1, kvh = 10, hd = 128, W = 8, P = 4, heads = 10, row = kvh * hd;
    cuda::GpuRSWACache g(L, kvh, hd, W);
    orc_cache* o = orc_cache_create(L, kvh, hd, W);
    g.reset(P);
    orc_cache_reset(o, P);
    auto pk = rvec(P * row), pv = rvec(P * row);
    float *dk = dev(pk), *dv = dev(pv);
    g.write_prefill(0, dk, dv, P);
    orc_cache_write_prefill(o, 0, pk.data(), pv.data(), P);
    // causal prefill attention (tests/test_rswa_cuda.cu:176-221 scenario)
    auto qa = rvec(P * heads * hd);
    float* dqa = dev(qa);
    float* douta = nullptr;
    cudaMalloc(&douta, qa.size() * 4);
    g.attention(0, dqa, P, 0, douta, heads, true);
    std::vector<float> wanta(qa.size());
    orc_cache_attention(o, 0, qa.data(), P, 0, wanta.data(), heads, 1);
    EXPECT(max_abs_diff(host(douta, qa.size()), wanta.data()) < 2e-5f);
    for (int t = 0; t < 24; ++t) {
        auto k = rvec(row), v = rvec(row);
        cudaMemcpy(dk, k.data(), row * 4, cudaMemcpyHostToDevice);
        cudaMemcpy(dv, v.data(), row * 4, cudaMemcpyHostToDevice);
        if (t % 2) g.append_decode(0, dk, dv); else g.append_decode_device(0, dk, dv);
        orc_cache_append_decode(o, 0, k.data(), v.data());
    }
    EXPECT(g.len(0) == orc_cache_len(o, 0));
    EXPECT(host(g.len_dev(0), 1)[0] == orc_cache_len(o, 0));
    const size_t n = static_cast<size_t>(g.capacity()) * row;
    EXPECT(std::memcmp(host(g.keys(0), n).data(), orc_cache_keys(o, 0), n * 4) == 0);
    EXPECT(std::memcmp(host(g.values(0), n).data(), orc_cache_values(o, 0), n * 4) == 0);
    auto q = rvec(heads * hd);
    float* dq = dev(q);
    float* dout = nullptr;
    cudaMalloc(&dout, q.size() * 4);
    g.attention(0, dq, 1, g.len(0) - 1, dout, heads, false);
    std::vector<float> want(q.size());
    orc_cache_attention(o, 0, q.data(), 1, orc_cache_len(o, 0) - 1, want.data(), heads, 0);
    EXPECT(max_abs_diff(host(dout, q.size()), want.data()) < 2e-5f);
    cudaFree(dk); cudaFree(dv); cudaFree(dqa); cudaFree(douta); cudaFree(dq); cudaFree(dout);
    orc_cache_destroy(o);
}

// ---- the reference's free functions, reference layout ----------------------------------------------------
static void test_free_functions_reference_layout() {
    std::printf("uocr::cuda::rswa_* (reference signatures, contiguous fp32 caches)\n");
    const int kvh = 4, heads = 4, hd = 64, W = 8, batch = 3, cap = 6 + W, row = kvh * hd;
    const int prefill[batch] = {4, 6, 3};
    const int slots[batch] = {2, 1, 0};
    std::vector<float> kb(static_cast<size_t>(batch) * cap * row, 0.f), vb(kb.size(), 0.f);
    orc_cache* o[batch];
    for (int s = 0; s < batch; ++s) {
        o[s] = orc_cache_create(1, kvh, hd, W);
        orc_cache_reset(o[s], prefill[s]);
        auto k = rvec(prefill[s] * row), v = rvec(prefill[s] * row);
        orc_cache_write_prefill(o[s], 0, k.data(), v.data(), prefill[s]);
        std::copy(k.begin(), k.end(), kb.begin() + static_cast<size_t>(s) * cap * row);
        std::copy(v.begin(), v.end(), vb.begin() + static_cast<size_t>(s) * cap * row);
    }
    float *dkb = dev(kb), *dvb = dev(vb);
    std::vector<int> len(prefill, prefill + batch), zero(batch, 0), sl(slots, slots + batch);
    int *d_len = dev(len), *d_ring = dev(zero), *d_pref = dev(len), *d_slots = dev(sl);
    float *dk, *dv, *dq, *dout;
    cudaMalloc(&dk, batch * row * 4); cudaMalloc(&dv, batch * row * 4);
    cudaMalloc(&dq, batch * heads * hd * 4); cudaMalloc(&dout, batch * heads * hd * 4);
    float worst = 0.f;
    for (int step = 0; step < 3 * W; ++step) {
        auto k = rvec(batch * row), v = rvec(batch * row), q = rvec(batch * heads * hd);
        cudaMemcpy(dk, k.data(), k.size() * 4, cudaMemcpyHostToDevice);
        cudaMemcpy(dv, v.data(), v.size() * 4, cudaMemcpyHostToDevice);
        cudaMemcpy(dq, q.data(), q.size() * 4, cudaMemcpyHostToDevice);
        cuda::rswa_append_decode_batch(dk, dv, dkb, dvb, d_len, d_ring, d_pref, d_slots, batch, cap, W, kvh, hd);
        cuda::rswa_attention_batch(dq, dkb, dvb, d_len, d_slots, batch, cap, heads, kvh, hd, dout);
        auto got = host(dout, q.size());
        for (int r = 0; r < batch; ++r) {
            orc_cache* c = o[slots[r]];
            orc_cache_append_decode(c, 0, k.data() + r * row, v.data() + r * row);
            std::vector<float> want(heads * hd);
            orc_cache_attention(c, 0, q.data() + r * heads * hd, 1, orc_cache_len(c, 0) - 1, want.data(), heads, 0);
            for (int i = 0; i < heads * hd; ++i) worst = std::max(worst, std::fabs(want[i] - got[r * heads * hd + i]));
        }
    }
    EXPECT(worst < 2e-5f);
    auto fk = host(dkb, kb.size()), fv = host(dvb, vb.size());
    auto flen = host(d_len, batch), fring = host(d_ring, batch);
    for (int s = 0; s < batch; ++s) {
        const size_t n = static_cast<size_t>(orc_cache_len(o[s], 0)) * row;
        EXPECT(flen[s] == orc_cache_len(o[s], 0) && fring[s] == orc_cache_ring_pos(o[s], 0));
        EXPECT(std::memcmp(fk.data() + static_cast<size_t>(s) * cap * row, orc_cache_keys(o[s], 0), n * 4) == 0);
        EXPECT(std::memcmp(fv.data() + static_cast<size_t>(s) * cap * row, orc_cache_values(o[s], 0), n * 4) == 0);
        orc_cache_destroy(o[s]);
    }
    // single-cache decode entry point (rswa_attention_decode) on slot 0's cache
    auto q1 = rvec(heads * hd);
    cudaMemcpy(dq, q1.data(), q1.size() * 4, cudaMemcpyHostToDevice);
    cuda::rswa_attention_decode(dq, dkb, dvb, flen[0], heads, kvh, hd, dout);
    cuda::rswa_attention_devlen(dq, dkb, dvb, d_len, 1, 0, heads, kvh, hd, false, dout + heads * hd);
    auto two = host(dout, 2 * heads * hd);
    EXPECT(std::memcmp(two.data(), two.data() + heads * hd, heads * hd * 4) == 0);
}

// ---- PagedBatchKV + SlotAllocator ---------------------------------------------------------------------------
static void test_paged_batch_kv() {
    std::printf("cuda::PagedBatchKV + SlotAllocator\n");
    SlotAllocator sa(4);
    EXPECT(sa.acquire(100) == 3 && sa.acquire(101) == 2 && sa.acquire(102) == 1);
    sa.release(101);
    EXPECT(sa.acquire(103) == 2 && sa.slot_of(103) == 2 && sa.slot_of(101) == -1);
    EXPECT(sa.acquire(104) == 0);
    bool threw = false;
    try { sa.acquire(105); } catch (const Error&) { threw = true; }
    EXPECT(threw);

    cuda::PagedBatchKV kv;
    cuda::PagedBatchKV::Config cfg;
    cfg.slots = 4; cfg.layers = 2; cfg.kv_heads = 2; cfg.head_dim = 16; cfg.window = 16;
    cfg.max_prefix_tokens = 40; cfg.prefix_arena_blocks = 4; cfg.ring_arena_blocks = 4; cfg.dtype = DType::BF16;
    EXPECT(kv.configure(cfg) == true);
    EXPECT(kv.configure(cfg) == false);  // same shape: buffers reused, state cleared
    const int row = cfg.kv_heads * cfg.head_dim, heads = 4, cap = cfg.max_prefix_tokens + cfg.window;
    const int P[4] = {33, 33, 16, 0};
    const char* keys[4] = {"docA", "docA", "docB", ""};
    orc_cache* o[4];
    for (int s = 0; s < 4; ++s) {
        auto a = kv.admit(s, keys[s], P[s]);
        EXPECT(a.prefix_is_new == (s == 0 || s == 2));
        if (s == 1) EXPECT(a.prefix_refcount == 2);
        o[s] = orc_cache_create(cfg.layers, cfg.kv_heads, cfg.head_dim, cfg.window);
        orc_cache_reset(o[s], P[s]);
    }
    EXPECT(kv.table_row(0)[0] == kv.table_row(1)[0] && kv.table_row(0)[2] == kv.table_row(1)[2]);  // shared prefix
    EXPECT(kv.table_row(0)[3] != kv.table_row(1)[3]);                                              // private rings
    EXPECT(kv.blocks().stats().live_prefixes == 2 && kv.blocks().shared_prefix_bytes() == 3 * 256);
    threw = false;
    try { cuda::PagedBatchKV::Admission x = kv.admit(0, "docC", 8); (void)x; } catch (const Error&) { threw = true; }
    EXPECT(threw);  // slot already bound

    // prefixes are written once, through the slot that created them; bf16 pool -> oracle gets rounded values
    auto round = [](std::vector<float> v) { for (auto& x : v) x = bf16_to_f32(f32_to_bf16(x)); return v; };
    for (int l = 0; l < cfg.layers; ++l)
        for (int s : {0, 2}) {
            auto k = round(rvec(P[s] * row)), v = round(rvec(P[s] * row));
            std::vector<int> rs(P[s], s), pos(P[s]);
            for (int i = 0; i < P[s]; ++i) pos[i] = i;
            float *dk = dev(k), *dv = dev(v);
            int *drs = dev(rs), *dpos = dev(pos);
            kv.write_prefill_ragged(l, dk, dv, drs, dpos, P[s]);
            cudaDeviceSynchronize();
            cudaFree(dk); cudaFree(dv); cudaFree(drs); cudaFree(dpos);
            for (int t = 0; t < 4; ++t)
                if (std::string(keys[t]) == keys[s] && P[t] == P[s]) orc_cache_write_prefill(o[t], l, k.data(), v.data(), P[s]);
        }
    std::vector<int> order = {2, 0, 3, 1};
    int* d_slots = dev(order);
    float *dq, *dk, *dv, *dout, *gk, *gv;
    cudaMalloc(&dq, 4 * heads * cfg.head_dim * 4); cudaMalloc(&dout, 4 * heads * cfg.head_dim * 4);
    cudaMalloc(&dk, 4 * row * 4); cudaMalloc(&dv, 4 * row * 4);
    cudaMalloc(&gk, 4 * cap * row * 4); cudaMalloc(&gv, 4 * cap * row * 4);
    float worst = 0.f;
    for (int t = 0; t < 2 * cfg.window + 5; ++t)
        for (int l = 0; l < cfg.layers; ++l) {
            auto k = round(rvec(4 * row)), v = round(rvec(4 * row)), q = rvec(4 * heads * cfg.head_dim);
            cudaMemcpy(dk, k.data(), k.size() * 4, cudaMemcpyHostToDevice);
            cudaMemcpy(dv, v.data(), v.size() * 4, cudaMemcpyHostToDevice);
            cudaMemcpy(dq, q.data(), q.size() * 4, cudaMemcpyHostToDevice);
            if (t % 2) {
                kv.decode_step(l, dq, dk, dv, d_slots, 4, heads, dout);
            } else {
                kv.append_decode_batch(l, dk, dv, d_slots, 4);
                kv.attention_batch(l, dq, d_slots, 4, heads, dout);
            }
            auto got = host(dout, q.size());
            for (int r = 0; r < 4; ++r) {
                orc_cache* c = o[order[r]];
                orc_cache_append_decode(c, l, k.data() + r * row, v.data() + r * row);
                std::vector<float> want(heads * cfg.head_dim);
                orc_cache_attention(c, l, q.data() + r * heads * cfg.head_dim, 1, orc_cache_len(c, l) - 1, want.data(), heads, 0);
                for (size_t i = 0; i < want.size(); ++i)
                    worst = std::max(worst, std::fabs(want[i] - got[r * heads * cfg.head_dim + i]));
            }
        }
    EXPECT(worst < 2e-5f);
    std::vector<int> ident = {0, 1, 2, 3};
    int* d_ident = dev(ident);
    for (int l = 0; l < cfg.layers; ++l) {
        kv.gather(l, d_ident, 4, gk, gv);
        auto hk = host(gk, static_cast<size_t>(4) * cap * row), hv = host(gv, static_cast<size_t>(4) * cap * row);
        auto dl = host(kv.d_len(l), 4), dr = host(kv.d_ring_pos(l), 4);
        for (int s = 0; s < 4; ++s) {
            const size_t n = static_cast<size_t>(orc_cache_len(o[s], l)) * row;
            EXPECT(dl[s] == orc_cache_len(o[s], l) && dr[s] == orc_cache_ring_pos(o[s], l));
            EXPECT(std::memcmp(hk.data() + static_cast<size_t>(s) * cap * row, orc_cache_keys(o[s], l), n * 4) == 0);
            EXPECT(std::memcmp(hv.data() + static_cast<size_t>(s) * cap * row, orc_cache_values(o[s], l), n * 4) == 0);
        }
    }
    EXPECT(kv.device_status() == 0);
    // releases: refcount drops, prefix freed with its last user, everything back to zero at the end
    kv.release(0);
    EXPECT(kv.blocks().stats().live_prefixes == 2 && kv.blocks().shared_prefix_bytes() == 0);
    kv.release(1);
    EXPECT(kv.blocks().stats().live_prefixes == 1);
    kv.release(1);  // releasing twice is harmless
    kv.release(2);
    kv.release(3);
    auto st = kv.blocks().stats();
    EXPECT(st.live_prefixes == 0 && st.prefix_live_bytes == 0 && st.ring_live_bytes == 0);
    // exhaustion: four rings fit, a fifth admission (after re-binding all slots) cannot happen; a too
    // large prefix set throws and leaves the arenas untouched
    kv.admit(0, "big1", 40);
    threw = false;
    try { kv.admit(1, "big2", 40); } catch (const Error&) { threw = true; }  // 3 + 3 blocks > 4
    EXPECT(threw);
    EXPECT(kv.blocks().stats().live_prefixes == 1 && kv.blocks().stats().ring_live_bytes == 256);
    for (int s = 0; s < 4; ++s) orc_cache_destroy(o[s]);
}

// ---- windowed ragged prefill through the host class: oracle by composition of reference calls ----------
static void test_windowed_prefill(bool tensor_cores) {
    std::printf("cuda::PagedBatchKV windowed prefill (%s)\n", tensor_cores ? "tcgen05 path" : "CUDA-core path");
    cuda::PagedBatchKV kv;
    cuda::PagedBatchKV::Config cfg;
    cfg.slots = 3; cfg.layers = 2; cfg.kv_heads = 2; cfg.dtype = DType::BF16;
    cfg.head_dim = tensor_cores ? 128 : 16;
    cfg.window = tensor_cores ? 160 : 16;
    cfg.max_prefix_tokens = tensor_cores ? 200 : 40;
    cfg.prefix_arena_blocks = 32; cfg.ring_arena_blocks = 3 * ((cfg.window + 15) / 16);
    kv.configure(cfg);
    const int heads = 4, row = cfg.kv_heads * cfg.head_dim, qrow = heads * cfg.head_dim;
    const int cap = cfg.max_prefix_tokens + cfg.window;
    // slot 2 and slot 0 share document A (slot 2 prefills it); slot 1 has its own; text shorter and longer than W
    const int P[3] = {tensor_cores ? 150 : 33, tensor_cores ? 200 : 16, tensor_cores ? 150 : 33};
    const int T[3] = {tensor_cores ? 70 : 9, tensor_cores ? 300 : 37, tensor_cores ? 401 : 50};
    const char* keys[3] = {"docA", "docB", "docA"};
    const int order[3] = {2, 1, 0};
    std::vector<cuda::PagedBatchKV::WindowedPrefill> reqs;
    for (int i = 0; i < 3; ++i) {
        const int sl = order[i];
        auto a = kv.admit(sl, keys[sl], P[sl]);
        reqs.push_back({sl, a.prefix_is_new ? P[sl] : 0, T[sl]});
    }
    EXPECT(reqs[0].vision_rows == P[2] && reqs[1].vision_rows == P[1] && reqs[2].vision_rows == 0);
    const int total = kv.plan_windowed_prefill(reqs);
    int nv = 0, nt = 0;
    for (auto& r : reqs) { nv += r.vision_rows; nt += r.text_rows; }
    EXPECT(total == nv + nt);
    auto round = [](std::vector<float> v) { for (auto& x : v) x = bf16_to_f32(f32_to_bf16(x)); return v; };
    orc_cache* o[3];
    for (int sl = 0; sl < 3; ++sl) {
        o[sl] = orc_cache_create(cfg.layers, cfg.kv_heads, cfg.head_dim, cfg.window);
        orc_cache_reset(o[sl], P[sl]);
    }
    float *dq, *dk, *dv, *dout;
    cudaMalloc(&dq, (size_t)total * qrow * 4); cudaMalloc(&dout, (size_t)total * qrow * 4);
    cudaMalloc(&dk, (size_t)total * row * 4); cudaMalloc(&dv, (size_t)total * row * 4);
    float worst = 0.f;
    for (int l = 0; l < cfg.layers; ++l) {
        auto q = rvec((size_t)total * qrow), k = round(rvec((size_t)total * row)), v = round(rvec((size_t)total * row));
        cudaMemcpy(dq, q.data(), q.size() * 4, cudaMemcpyHostToDevice);
        cudaMemcpy(dk, k.data(), k.size() * 4, cudaMemcpyHostToDevice);
        cudaMemcpy(dv, v.data(), v.size() * 4, cudaMemcpyHostToDevice);
        cudaMemset(dout, 0xff, (size_t)total * qrow * 4);
        kv.windowed_prefill_layer(l, dq, dk, dv, heads, dout);
        auto got = host(dout, (size_t)total * qrow);
        // oracle: vision rows causal over the prefix (the sharing slot gets the same prefix without queries)
        std::vector<float> want((size_t)total * qrow, 0.f);
        int at = 0;
        for (auto& r : reqs) {
            if (r.vision_rows == 0) continue;
            for (int sl = 0; sl < 3; ++sl)
                if (std::string(keys[sl]) == keys[r.slot])
                    orc_cache_write_prefill(o[sl], l, k.data() + (size_t)at * row, v.data() + (size_t)at * row, r.vision_rows);
            orc_cache_attention(o[r.slot], l, q.data() + (size_t)at * qrow, r.vision_rows, 0, want.data() + (size_t)at * qrow, heads, 1);
            at += r.vision_rows;
        }
        for (auto& r : reqs) {  // text rows: append, then attend everything cached
            for (int i = 0; i < r.text_rows; ++i, ++at) {
                orc_cache_append_decode(o[r.slot], l, k.data() + (size_t)at * row, v.data() + (size_t)at * row);
                orc_cache_attention(o[r.slot], l, q.data() + (size_t)at * qrow, 1, orc_cache_len(o[r.slot], l) - 1,
                                    want.data() + (size_t)at * qrow, heads, 0);
            }
        }
        worst = std::max(worst, max_abs_diff(want, got.data()));
    }
    std::printf("  max abs difference %.3g\n", worst);
    EXPECT(worst < (tensor_cores ? 2e-4f : 2e-5f));
    // cursors and logical cache contents are those of the appends, bit for bit
    std::vector<int> ident = {0, 1, 2};
    int* d_ident = dev(ident);
    float *gk, *gv;
    cudaMalloc(&gk, (size_t)3 * cap * row * 4); cudaMalloc(&gv, (size_t)3 * cap * row * 4);
    for (int l = 0; l < cfg.layers; ++l) {
        kv.gather(l, d_ident, 3, gk, gv);
        auto hk = host(gk, (size_t)3 * cap * row), hv = host(gv, (size_t)3 * cap * row);
        auto dl = host(kv.d_len(l), 3), dr = host(kv.d_ring_pos(l), 3);
        for (int sl = 0; sl < 3; ++sl) {
            const size_t n = (size_t)orc_cache_len(o[sl], l) * row;
            EXPECT(dl[sl] == orc_cache_len(o[sl], l) && dr[sl] == orc_cache_ring_pos(o[sl], l));
            EXPECT(std::memcmp(hk.data() + (size_t)sl * cap * row, orc_cache_keys(o[sl], l), n * 4) == 0);
            EXPECT(std::memcmp(hv.data() + (size_t)sl * cap * row, orc_cache_values(o[sl], l), n * 4) == 0);
        }
    }
    EXPECT(kv.device_status() == 0);
    if (!tensor_cores) {
        // snapshot of slot 1 in the reference's export format: [kv_heads, len, head_dim] fp32 per layer
        const char* env = std::getenv("UOCR_SNAPSHOT_DIR");
        const std::string dir = env ? env : "/tmp";
        kv.export_snapshot(dir, 1, "final");
        for (int l = 0; l < cfg.layers; ++l) {
            const int n = orc_cache_len(o[1], l);
            for (int which = 0; which < 2; ++which) {
                const std::string path = dir + "/final_" + (which ? "v_" : "k_") + std::to_string(l) + ".bin";
                std::vector<float> file((size_t)cfg.kv_heads * n * cfg.head_dim);
                FILE* f = std::fopen(path.c_str(), "rb");
                EXPECT(f != nullptr);
                if (!f) continue;
                EXPECT(std::fread(file.data(), 4, file.size(), f) == file.size());
                EXPECT(std::fgetc(f) == EOF);
                std::fclose(f);
                const float* want = which ? orc_cache_values(o[1], l) : orc_cache_keys(o[1], l);
                bool same = true;
                for (int h = 0; h < cfg.kv_heads && same; ++h)
                    for (int t = 0; t < n && same; ++t)
                        same = std::memcmp(&file[((size_t)h * n + t) * cfg.head_dim],
                                           want + ((size_t)t * cfg.kv_heads + h) * cfg.head_dim, cfg.head_dim * 4) == 0;
                EXPECT(same);
            }
        }
    }
    for (int sl = 0; sl < 3; ++sl) orc_cache_destroy(o[sl]);
    cudaFree(dq); cudaFree(dk); cudaFree(dv); cudaFree(dout); cudaFree(gk); cudaFree(gv); cudaFree(d_ident);
}

// ---- GpuRSWACache inside a captured graph: device cursors, device-length attention ----------------------------
static void test_gpu_cache_graph_replay() {
    std::printf("cuda::GpuRSWACache: captured append_decode_device + attention_devlen, replayed across the ring boundary\n");
    const int kvh = 2, hd = 64, W = 8, P = 5, heads = 4, row = kvh * hd;
    cuda::GpuRSWACache g(1, kvh, hd, W);
    orc_cache* o = orc_cache_create(1, kvh, hd, W);
    g.reset(P);
    orc_cache_reset(o, P);
    auto pk = rvec(P * row), pv = rvec(P * row);
    float *dpk = dev(pk), *dpv = dev(pv);
    g.write_prefill(0, dpk, dpv, P);
    orc_cache_write_prefill(o, 0, pk.data(), pv.data(), P);
    g.reset_device_state(P);
    float *dk, *dv, *dq, *dout;
    cudaMalloc(&dk, row * 4); cudaMalloc(&dv, row * 4); cudaMalloc(&dq, heads * hd * 4); cudaMalloc(&dout, heads * hd * 4);
    cudaStream_t st;
    cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking);
    // one plain step first (kernel attributes, and the same call sequence the graph will hold)
    auto step_inputs = [&](std::vector<float>& k, std::vector<float>& v, std::vector<float>& q) {
        k = rvec(row); v = rvec(row); q = rvec(heads * hd);
        cudaMemcpyAsync(dk, k.data(), row * 4, cudaMemcpyHostToDevice, st);
        cudaMemcpyAsync(dv, v.data(), row * 4, cudaMemcpyHostToDevice, st);
        cudaMemcpyAsync(dq, q.data(), heads * hd * 4, cudaMemcpyHostToDevice, st);
        cudaStreamSynchronize(st);
    };
    std::vector<float> k, v, q;
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal);
    bool threw = false;
    try { g.keys(0, st); } catch (const Error&) { threw = true; }  // a snapshot inside capture is refused
    EXPECT(threw);
    g.append_decode_device(0, dk, dv, st);
    g.attention_devlen(0, dq, 1, 0, dout, heads, false, st);
    EXPECT(cudaStreamEndCapture(st, &graph) == cudaSuccess);
    EXPECT(cudaGraphInstantiate(&exec, graph, nullptr, nullptr, 0) == cudaSuccess);
    float worst = 0.f;
    for (int t = 0; t < 3 * W + 2; ++t) {
        step_inputs(k, v, q);
        EXPECT(cudaGraphLaunch(exec, st) == cudaSuccess);
        cudaStreamSynchronize(st);
        orc_cache_append_decode(o, 0, k.data(), v.data());
        std::vector<float> want(heads * hd);
        orc_cache_attention(o, 0, q.data(), 1, orc_cache_len(o, 0) - 1, want.data(), heads, 0);
        worst = std::max(worst, max_abs_diff(host(dout, heads * hd), want.data()));
        EXPECT(host(g.len_dev(0), 1)[0] == orc_cache_len(o, 0));
    }
    EXPECT(worst < 2e-5f);
    const size_t n = static_cast<size_t>(orc_cache_len(o, 0)) * row;
    EXPECT(std::memcmp(host(g.keys(0, st), n).data(), orc_cache_keys(o, 0), n * 4) == 0);  // outside capture: allowed
    EXPECT(std::memcmp(host(g.values(0, st), n).data(), orc_cache_values(o, 0), n * 4) == 0);
    cudaGraphExecDestroy(exec); cudaGraphDestroy(graph); cudaStreamDestroy(st);
    cudaFree(dpk); cudaFree(dpv); cudaFree(dk); cudaFree(dv); cudaFree(dq); cudaFree(dout);
    orc_cache_destroy(o);
}

// ---- the reference-signature wrappers under capture: prepared scratch, never reallocated -----------------------
static void test_free_functions_capture_and_scratch_rules() {
    std::printf("uocr::cuda::rswa_* inside stream capture (prepared per-stream scratch)\n");
    const int kvh = 2, heads = 2, hd = 32, W = 8, batch = 2, cap = 4 + W, row = kvh * hd;
    std::vector<float> kb = rvec(static_cast<size_t>(batch) * cap * row), vb = rvec(kb.size());
    float *dkb = dev(kb), *dvb = dev(vb);
    std::vector<int> len = {7, 12}, sl = {1, 0};
    int *d_len = dev(len), *d_slots = dev(sl);
    auto q = rvec(batch * heads * hd);
    float* dq = dev(q);
    float *dout, *dref;
    cudaMalloc(&dout, q.size() * 4); cudaMalloc(&dref, q.size() * 4);
    cudaStream_t st;
    cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking);
    EXPECT(cuda::rswa_prepare(st, 64));
    cuda::rswa_attention_batch(dq, dkb, dvb, d_len, d_slots, batch, cap, heads, kvh, hd, dref, st);  // plain call
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal);
    cuda::rswa_attention_batch(dq, dkb, dvb, d_len, d_slots, batch, cap, heads, kvh, hd, dout, st);
    EXPECT(cudaStreamEndCapture(st, &graph) == cudaSuccess);
    EXPECT(cudaGraphInstantiate(&exec, graph, nullptr, nullptr, 0) == cudaSuccess);
    // a call with more rows than were prepared launches nothing (and frees nothing): the graph stays valid
    cudaMemset(dout, 0xff, q.size() * 4);
    std::vector<int> many_slots(100, 0);
    int* d_many = dev(many_slots);
    cuda::rswa_attention_batch(dq, dkb, dvb, d_len, d_many, 100, cap, heads, kvh, hd, dout, st);  // prints the refusal
    cudaStreamSynchronize(st);
    auto untouched = host(dout, q.size());
    bool all_nan = true;
    for (float x : untouched) all_nan = all_nan && std::isnan(x);
    EXPECT(all_nan);
    EXPECT(cuda::rswa_prepare(st, 256));  // larger scratch for later calls; the old one stays alive for the graph
    EXPECT(cudaGraphLaunch(exec, st) == cudaSuccess);
    cudaStreamSynchronize(st);
    auto a = host(dout, q.size()), b = host(dref, q.size());
    EXPECT(std::memcmp(a.data(), b.data(), a.size() * 4) == 0);
    // another stream gets scratch of its own
    cudaStream_t st2;
    cudaStreamCreateWithFlags(&st2, cudaStreamNonBlocking);
    cudaMemsetAsync(dout, 0, q.size() * 4, st2);
    cuda::rswa_attention_batch(dq, dkb, dvb, d_len, d_slots, batch, cap, heads, kvh, hd, dout, st2);
    cudaStreamSynchronize(st2);
    a = host(dout, q.size());
    EXPECT(std::memcmp(a.data(), b.data(), a.size() * 4) == 0);
    cudaGraphExecDestroy(exec); cudaGraphDestroy(graph); cudaStreamDestroy(st); cudaStreamDestroy(st2);
    cudaFree(dkb); cudaFree(dvb); cudaFree(d_len); cudaFree(d_slots); cudaFree(dq); cudaFree(dout); cudaFree(dref); cudaFree(d_many);
}

// ---- admission waves, captured decode steps and the GpuDecoder-named adapter -----------------------------------
static void test_decoder_kv_adapter_waves_and_step_graphs() {
    std::printf("cuda::GpuDecoderKV: batch_prefill (one state upload per wave), batch_decode graphs, release\n");
    const int L = 3, kvh = 2, hd = 32, W = 16, heads = 4, row = kvh * hd, qrow = heads * hd, slots = 4;
    const int capacity = 40 + W;
    cuda::GpuDecoderKV dec(L, kvh, hd, W, DType::BF16);
    EXPECT(dec.batch_configure(slots, capacity) == true);
    EXPECT(dec.batch_configure(slots, capacity) == false);
    EXPECT(dec.batch_slots() == slots && dec.batch_graph_count() == 0);
    cudaStream_t st;
    cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking);
    auto round = [](std::vector<float> v) { for (auto& x : v) x = bf16_to_f32(f32_to_bf16(x)); return v; };
    // wave of three requests: prompts of 21, 7 and 33 tokens into slots 3, 0, 2 (the whole prompt is the fixed region)
    const std::vector<int> lengths = {21, 7, 33}, pslots = {3, 0, 2};
    std::vector<int> starts = {0, 21, 28};
    const int total = dec.batch_prefill_begin(starts, lengths, pslots, {}, st);
    EXPECT(total == 61);
    orc_cache* o[slots] = {nullptr, nullptr, nullptr, nullptr};
    for (size_t r = 0; r < lengths.size(); ++r) {
        o[pslots[r]] = orc_cache_create(L, kvh, hd, W);
        orc_cache_reset(o[pslots[r]], lengths[r]);
    }
    float *dq, *dk, *dv, *dctx;
    cudaMalloc(&dq, (size_t)L * total * qrow * 4); cudaMalloc(&dctx, (size_t)L * total * qrow * 4);
    cudaMalloc(&dk, (size_t)L * total * row * 4); cudaMalloc(&dv, (size_t)L * total * row * 4);
    float worst = 0.f;
    for (int l = 0; l < L; ++l) {
        auto q = rvec((size_t)total * qrow), k = round(rvec((size_t)total * row)), v = round(rvec((size_t)total * row));
        cudaMemcpyAsync(dq, q.data(), q.size() * 4, cudaMemcpyHostToDevice, st);
        cudaMemcpyAsync(dk, k.data(), k.size() * 4, cudaMemcpyHostToDevice, st);
        cudaMemcpyAsync(dv, v.data(), v.size() * 4, cudaMemcpyHostToDevice, st);
        dec.attention_block_ragged(l, dq, dk, dv, dctx, total, heads, st);
        cudaStreamSynchronize(st);
        auto got = host(dctx, (size_t)total * qrow);
        for (size_t r = 0; r < lengths.size(); ++r) {
            orc_cache* c = o[pslots[r]];
            orc_cache_write_prefill(c, l, k.data() + (size_t)starts[r] * row, v.data() + (size_t)starts[r] * row, lengths[r]);
            std::vector<float> want((size_t)lengths[r] * qrow);
            orc_cache_attention(c, l, q.data() + (size_t)starts[r] * qrow, lengths[r], 0, want.data(), heads, 1);
            worst = std::max(worst, max_abs_diff(want, got.data() + (size_t)starts[r] * qrow));
        }
    }
    EXPECT(worst < 2e-5f);
    // decode: batch of 3, fixed activation buffers [L][batch][row], one graph per batch size
    const int batch = 3;
    const std::vector<int> order = {2, 3, 0};
    cuda::PagedBatchKV::StepIO io;
    io.q = dq; io.k = dk; io.v = dv; io.out = dctx; io.heads = heads;
    io.q_layer_stride = (long long)batch * qrow; io.kv_layer_stride = (long long)batch * row; io.out_layer_stride = (long long)batch * qrow;
    worst = 0.f;
    for (int t = 0; t < 2 * W + 3; ++t) {
        auto q = rvec((size_t)L * batch * qrow), k = round(rvec((size_t)L * batch * row)), v = round(rvec((size_t)L * batch * row));
        cudaMemcpyAsync(dq, q.data(), q.size() * 4, cudaMemcpyHostToDevice, st);
        cudaMemcpyAsync(dk, k.data(), k.size() * 4, cudaMemcpyHostToDevice, st);
        cudaMemcpyAsync(dv, v.data(), v.size() * 4, cudaMemcpyHostToDevice, st);
        dec.batch_decode({}, order, io, false, st);
        cudaStreamSynchronize(st);
        auto got = host(dctx, (size_t)L * batch * qrow);
        for (int l = 0; l < L; ++l)
            for (int r = 0; r < batch; ++r) {
                orc_cache* c = o[order[r]];
                orc_cache_append_decode(c, l, k.data() + ((size_t)l * batch + r) * row, v.data() + ((size_t)l * batch + r) * row);
                std::vector<float> want(qrow);
                orc_cache_attention(c, l, q.data() + ((size_t)l * batch + r) * qrow, 1, orc_cache_len(c, l) - 1, want.data(), heads, 0);
                worst = std::max(worst, max_abs_diff(want, got.data() + ((size_t)l * batch + r) * qrow));
            }
    }
    EXPECT(worst < 2e-5f);
    EXPECT(dec.batch_graph_count() == 1);  // captured once, replayed across the warm-up -> ring boundary
    // cursors and contents after the replays, bit for bit
    const int cap = capacity;
    std::vector<int> ident = {0, 1, 2, 3};
    int* d_ident = dev(ident);
    float *gk, *gv;
    cudaMalloc(&gk, (size_t)slots * cap * row * 4); cudaMalloc(&gv, (size_t)slots * cap * row * 4);
    for (int l = 0; l < L; ++l) {
        dec.kv().gather(l, d_ident, slots, gk, gv, st);
        cudaStreamSynchronize(st);
        auto hk = host(gk, (size_t)slots * cap * row), hv = host(gv, (size_t)slots * cap * row);
        auto dl = host(dec.kv().d_len(l), slots), dr = host(dec.kv().d_ring_pos(l), slots);
        for (int sl : {0, 2, 3}) {
            const size_t n = (size_t)orc_cache_len(o[sl], l) * row;
            EXPECT(dl[sl] == orc_cache_len(o[sl], l) && dr[sl] == orc_cache_ring_pos(o[sl], l));
            EXPECT(std::memcmp(hk.data() + (size_t)sl * cap * row, orc_cache_keys(o[sl], l), n * 4) == 0);
            EXPECT(std::memcmp(hv.data() + (size_t)sl * cap * row, orc_cache_values(o[sl], l), n * 4) == 0);
        }
    }
    // a second batch size gets its own graph; release poisons the slot's device row
    dec.batch_decode({}, {3, 0}, io, false, st);
    EXPECT(dec.batch_graph_count() == 2);
    dec.batch_release(2, st);
    cudaStreamSynchronize(st);
    auto row2 = host(dec.kv().layer_view(0).block_table + 2 * dec.kv().layer_view(0).table_stride, dec.kv().layer_view(0).table_stride);
    bool all_minus_one = true;
    for (int x : row2) all_minus_one = all_minus_one && x == -1;
    EXPECT(all_minus_one);
    EXPECT(host(dec.kv().d_len(1), slots)[2] == 0 && host(dec.kv().d_prefill_len(), slots)[2] == 0);
    EXPECT(dec.kv().device_status(st) == 0);
    dec.batch_decode({}, order, io, false, st);  // slot 2 is stale now: flagged, not obeyed
    EXPECT((dec.kv().device_status(st) & 1) != 0);
    // an all-or-nothing wave: the second request cannot be placed, the first is rolled back
    const auto before = dec.kv().blocks().stats();
    bool threw = false;
    try {
        dec.kv().admit_wave({{2, "docX", 8}, {1, "docY", capacity}}, st);  // prefix longer than configured
    } catch (const Error&) { threw = true; }
    EXPECT(threw);
    const auto after = dec.kv().blocks().stats();
    EXPECT(before.live_prefixes == after.live_prefixes && before.ring_live_bytes == after.ring_live_bytes);
    // a new shape reallocates and drops the captured graphs (src/engine/gpu_decoder.cu:929-931)
    EXPECT(dec.batch_configure(slots + 1, capacity) == true);
    EXPECT(dec.batch_graph_count() == 0);
    for (int sl : {0, 2, 3}) orc_cache_destroy(o[sl]);
    cudaStreamDestroy(st);
    cudaFree(dq); cudaFree(dk); cudaFree(dv); cudaFree(dctx); cudaFree(gk); cudaFree(gv); cudaFree(d_ident);
}

// ---- a packed prefill larger than the attention scratch is served in chunks -------------------------------------
static void test_large_ragged_prefill_is_chunked() {
    std::printf("cuda::GpuDecoderKV: ragged prefill of 4300 rows (scratch holds 4096 per call)\n");
    const int L = 1, kvh = 1, hd = 32, W = 16, heads = 2, row = kvh * hd, qrow = heads * hd;
    const int total = 4300;
    cuda::GpuDecoderKV dec(L, kvh, hd, W, DType::BF16);
    dec.batch_configure(2, total + W);
    cudaStream_t st;
    cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking);
    EXPECT(dec.batch_prefill_begin({0, 4000}, {4000, 300}, {1, 0}, {}, st) == total);
    auto round = [](std::vector<float> v) { for (auto& x : v) x = bf16_to_f32(f32_to_bf16(x)); return v; };
    auto q = rvec((size_t)total * qrow), k = round(rvec((size_t)total * row)), v = round(rvec((size_t)total * row));
    float *dq = dev(q), *dk = dev(k), *dv = dev(v), *dctx;
    cudaMalloc(&dctx, (size_t)total * qrow * 4);
    cudaMemset(dctx, 0xff, (size_t)total * qrow * 4);
    dec.attention_block_ragged(0, dq, dk, dv, dctx, total, heads, st);
    cudaStreamSynchronize(st);
    auto got = host(dctx, (size_t)total * qrow);
    float worst = 0.f;
    const int starts[2] = {0, 4000}, lens[2] = {4000, 300};
    for (int r = 0; r < 2; ++r) {
        orc_cache* c = orc_cache_create(L, kvh, hd, W);
        orc_cache_reset(c, lens[r]);
        orc_cache_write_prefill(c, 0, k.data() + (size_t)starts[r] * row, v.data() + (size_t)starts[r] * row, lens[r]);
        std::vector<float> want((size_t)lens[r] * qrow);
        orc_cache_attention(c, 0, q.data() + (size_t)starts[r] * qrow, lens[r], 0, want.data(), heads, 1);
        worst = std::max(worst, max_abs_diff(want, got.data() + (size_t)starts[r] * qrow));
        orc_cache_destroy(c);
    }
    EXPECT(worst < 2e-5f);
    EXPECT(dec.kv().device_status(st) == 0);
    cudaStreamDestroy(st);
    cudaFree(dq); cudaFree(dk); cudaFree(dv); cudaFree(dctx);
}

int main() {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0) {
        std::printf("no CUDA device\n");
        return 2;
    }
    try {
        test_rswa_cache_host_interface();
        test_gpu_cache_device_interface();
        test_free_functions_reference_layout();
        test_paged_batch_kv();
        test_windowed_prefill(false);
        test_windowed_prefill(true);
        test_gpu_cache_graph_replay();
        test_free_functions_capture_and_scratch_rules();
        test_decoder_kv_adapter_waves_and_step_graphs();
        test_large_ragged_prefill_is_chunked();
    } catch (const std::exception& e) {
        std::printf("  EXCEPTION: %s\n", e.what());
        ++g_fail;
    }
    std::printf("%s (%d failures)\n", g_fail ? "FAILED" : "ALL OK", g_fail);
    return g_fail ? 1 : 0;
}
