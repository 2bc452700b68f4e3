// extern "C" boundary of libuocr_rswa_b200.so: argument checking, geometry dispatch and kernel
// launches.  No entry point here allocates (except workspace_create), synchronises (except
// workspace_status) or falls back to host code.
#include <cuda_runtime.h>

#include <atomic>
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "rswa_attention.cuh"
#include "rswa_copy.cuh"
#include "rswa_prefill_tc.cuh"
#include "rswa_stream_read.cuh"
#include "uocr_rswa_b200.h"

using namespace uocr_b200;

namespace {

thread_local std::string g_last_error;
std::atomic<uint64_t> g_launches{0};

int fail(int code, const std::string& msg) {
    g_last_error = msg;
    return code;
}

int cuda_fail(cudaError_t e, const char* what) {
    return fail(UOCR_B200_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e));
}

#define CHECK_CUDA(expr, what)                             \
    do {                                                   \
        cudaError_t e_ = (expr);                           \
        if (e_ != cudaSuccess) return cuda_fail(e_, what); \
    } while (0)

int after_launch(const char* what) {
    g_launches.fetch_add(1, std::memory_order_relaxed);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, what);
    return UOCR_B200_OK;
}

struct DeviceInfo {
    bool known = false;
    int sms = 0;
    int smem_optin = 0;
    int cc_major = 0;
};
DeviceInfo g_dev[64];

int device_info(const DeviceInfo** out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(UOCR_B200_ERR_NO_DEVICE, std::string("cudaGetDevice: ") + cudaGetErrorString(e));
    if (dev < 0 || dev >= 64) return fail(UOCR_B200_ERR_NO_DEVICE, "device ordinal out of range");
    DeviceInfo& d = g_dev[dev];
    if (!d.known) {
        CHECK_CUDA(cudaDeviceGetAttribute(&d.sms, cudaDevAttrMultiProcessorCount, dev), "sm count");
        CHECK_CUDA(cudaDeviceGetAttribute(&d.smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev), "smem optin");
        CHECK_CUDA(cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, dev), "cc major");
        if (d.cc_major != 10)
            return fail(UOCR_B200_ERR_NO_DEVICE, "this library only carries sm_100a code (B200)");
        d.known = true;
    }
    *out = &d;
    return UOCR_B200_OK;
}

constexpr int kMaxWarpsPerCta = UOCR_ATTN_THREADS / 32;
constexpr int kMaxHeadDim = 256;

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

bool head_dim_ok(int hd, int dtype) {
    if (hd < (dtype == UOCR_B200_BF16 ? 8 : 4) || hd > kMaxHeadDim) return false;
    return (hd & (hd - 1)) == 0;
}

}  // namespace

// =================================================================================================
// workspace
// =================================================================================================
struct uocr_b200_workspace {
    int device = 0;
    int max_rows = 0;
    int total_warps_max = 0;
    uint8_t* base = nullptr;
    size_t bytes = 0;
    int* status = nullptr;
    int* rs = nullptr;
    RowInfo* info = nullptr;
    float* part_acc = nullptr;
    float* part_ml = nullptr;
    int* counters = nullptr;   // [pieces_max] arrival counters, zero between launches
    int* planned_ctas = nullptr;  // fused step: ticket counter of CTAs that have planned; wraps to zero by itself
    int pieces_max = 0;
    uint32_t wait_limit = kWaitLimit;  // polls a tile wait may take (uocr_b200_workspace_set_wait_limit)
    PrefillTile* tiles = nullptr;  // [max_rows] query-tile descriptors of the tensor-core prefill
    TcWork* tile_work = nullptr;   // [max_rows] the same tiles, most key tiles first, with their key-tile counts
    int* item_counter = nullptr;   // items the persistent prefill grid has handed out beyond every CTA's first
    int plan_tiles = 0;            // tiles of the plan in tile_work (0: none)
    int plan_window = 0;
    bool plan_any_text = false;
    unsigned plan_serial = 0;      // plans made on this workspace so far
    int tiles_cap = 0;
    bool out_bf16 = false;  // attention results are written as bf16 instead of fp32
    bool timing = false;
    bool overlap = false;  // fused decode step may start its prologue before the preceding kernel ends
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
};

extern "C" {

const char* uocr_b200_status_string(int s) {
    switch (s) {
        case UOCR_B200_OK: return "ok";
        case UOCR_B200_ERR_INVALID: return "invalid argument";
        case UOCR_B200_ERR_UNSUPPORTED: return "unsupported geometry";
        case UOCR_B200_ERR_CUDA: return "CUDA error";
        case UOCR_B200_ERR_WORKSPACE: return "workspace too small";
        case UOCR_B200_ERR_NO_DEVICE: return "no usable sm_100 device";
        case UOCR_B200_ERR_DEVICE_STATUS: return "device-side fault recorded";
        case UOCR_B200_ERR_EXHAUSTED: return "pool exhausted";
        default: return "unknown status";
    }
}

const char* uocr_b200_last_error(void) { return g_last_error.c_str(); }
const char* uocr_b200_version(void) { return "uocr_rswa_b200 0.1 sm_100a"; }
uint64_t uocr_b200_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int uocr_b200_workspace_create(int max_rows, uocr_b200_workspace** out) {
    if (!out || max_rows <= 0) return fail(UOCR_B200_ERR_INVALID, "workspace_create: bad arguments");
    const DeviceInfo* di = nullptr;
    if (int rc = device_info(&di)) return rc;
    auto* ws = new uocr_b200_workspace;
    cudaGetDevice(&ws->device);
    ws->max_rows = max_rows;
    ws->total_warps_max = di->sms * kMaxWarpsPerCta;
    auto up = [](size_t x) { return (x + 255) & ~size_t(255); };
    const size_t o_status = 0;
    const size_t o_rs = up(256);
    const size_t o_info = o_rs + up(sizeof(int) * (size_t)(max_rows + 1));
    ws->pieces_max = ws->total_warps_max;
    const size_t o_acc = o_info + up(sizeof(RowInfo) * (size_t)max_rows);
    const size_t o_ml = o_acc + up(sizeof(float) * 2 * (size_t)ws->pieces_max * kMaxHeadDim);
    const size_t o_cnt = o_ml + up(sizeof(float) * 4 * (size_t)ws->pieces_max);
    const size_t o_tiles = o_cnt + up(sizeof(int) * ((size_t)ws->pieces_max + 64));
    ws->tiles_cap = max_rows;
    const size_t o_order = o_tiles + up(sizeof(PrefillTile) * (size_t)ws->tiles_cap);
    ws->bytes = o_order + up(sizeof(TcWork) * (size_t)ws->tiles_cap) + 256;
    cudaError_t e = cudaMalloc(&ws->base, ws->bytes);
    if (e != cudaSuccess) {
        delete ws;
        return cuda_fail(e, "workspace cudaMalloc");
    }
    e = cudaMemset(ws->base, 0, ws->bytes);
    if (e != cudaSuccess) {
        cudaFree(ws->base);
        delete ws;
        return cuda_fail(e, "workspace cudaMemset");
    }
    ws->status = reinterpret_cast<int*>(ws->base + o_status);
    ws->rs = reinterpret_cast<int*>(ws->base + o_rs);
    ws->info = reinterpret_cast<RowInfo*>(ws->base + o_info);
    ws->part_acc = reinterpret_cast<float*>(ws->base + o_acc);
    ws->part_ml = reinterpret_cast<float*>(ws->base + o_ml);
    ws->counters = reinterpret_cast<int*>(ws->base + o_cnt);
    ws->planned_ctas = ws->counters + ws->pieces_max;
    ws->tiles = reinterpret_cast<PrefillTile*>(ws->base + o_tiles);
    ws->tile_work = reinterpret_cast<TcWork*>(ws->base + o_order);
    ws->item_counter = reinterpret_cast<int*>(ws->base + o_order + up(sizeof(TcWork) * (size_t)ws->tiles_cap));
    *out = ws;
    return UOCR_B200_OK;
}

int uocr_b200_workspace_destroy(uocr_b200_workspace* ws) {
    if (!ws) return UOCR_B200_OK;
    if (ws->base) cudaFree(ws->base);
    if (ws->ev0) cudaEventDestroy(ws->ev0);
    if (ws->ev1) cudaEventDestroy(ws->ev1);
    delete ws;
    return UOCR_B200_OK;
}

int uocr_b200_workspace_set_timing(uocr_b200_workspace* ws, int enabled) {
    if (!ws) return fail(UOCR_B200_ERR_INVALID, "workspace_set_timing: null workspace");
    if (enabled && !ws->ev0) {
        CHECK_CUDA(cudaEventCreate(&ws->ev0), "event create");
        CHECK_CUDA(cudaEventCreate(&ws->ev1), "event create");
    }
    ws->timing = enabled != 0;
    return UOCR_B200_OK;
}

int uocr_b200_workspace_stream_read_gbs(uocr_b200_workspace* ws, uocr_b200_stream_t stream, double* gbs) {
    if (!ws || !gbs) return fail(UOCR_B200_ERR_INVALID, "workspace_stream_read_gbs: null argument");
    const DeviceInfo* di = nullptr;
    if (int rc = device_info(&di)) return rc;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    // one CTA per SM, each walking its own 8 MB (the whole buffer, 1.2 GB, is far larger than L2) twice
    constexpr int kTilesPerCta = 2048, kPasses = 2, kRuns = 5, warps = 16;
    const int ctas = di->sms;
    const size_t bytes = (size_t)ctas * kTilesPerCta * kStreamTile;
    uint8_t* buf = nullptr;
    unsigned long long* d_out = nullptr;
    CHECK_CUDA(cudaMalloc(&buf, bytes), "streaming buffer");
    cudaError_t e = cudaMalloc(&d_out, sizeof(unsigned long long) * 2 * ctas);
    cudaEvent_t ev[2] = {nullptr, nullptr};
    if (e == cudaSuccess) e = cudaEventCreate(&ev[0]);
    if (e == cudaSuccess) e = cudaEventCreate(&ev[1]);
    const int smem = ((warps * kStreamRing * 8 + 127) & ~127) + warps * kStreamRing * kStreamTile;
    if (e == cudaSuccess) e = cudaFuncSetAttribute(rswa_stream_read_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e == cudaSuccess) e = cudaMemsetAsync(buf, 0, bytes, st);
    std::vector<float> ms;
    for (int r = 0; r < kRuns + 1 && e == cudaSuccess; ++r) {
        StreamReadParams cp{buf, kTilesPerCta, kPasses, d_out, ws->status};
        e = cudaEventRecord(ev[0], st);
        rswa_stream_read_kernel<<<ctas, warps * 32, smem, st>>>(cp);
        g_launches.fetch_add(1, std::memory_order_relaxed);
        if (e == cudaSuccess) e = cudaGetLastError();
        if (e == cudaSuccess) e = cudaEventRecord(ev[1], st);
        if (e == cudaSuccess) e = cudaEventSynchronize(ev[1]);
        float t = 0.f;
        if (e == cudaSuccess) e = cudaEventElapsedTime(&t, ev[0], ev[1]);
        if (r > 0) ms.push_back(t);  // the first run is the warm-up
    }
    cudaFree(buf);
    if (d_out) cudaFree(d_out);
    if (ev[0]) cudaEventDestroy(ev[0]);
    if (ev[1]) cudaEventDestroy(ev[1]);
    if (e != cudaSuccess) return cuda_fail(e, "streaming-rate run");
    std::sort(ms.begin(), ms.end());
    *gbs = (double)bytes * kPasses / (ms[ms.size() / 2] * 1e-3) / 1e9;
    return UOCR_B200_OK;
}

int uocr_b200_workspace_set_out_dtype(uocr_b200_workspace* ws, int dtype) {
    if (!ws) return fail(UOCR_B200_ERR_INVALID, "workspace_set_out_dtype: null workspace");
    if (dtype != UOCR_B200_F32 && dtype != UOCR_B200_BF16) return fail(UOCR_B200_ERR_UNSUPPORTED, "workspace_set_out_dtype: fp32 or bf16");
    ws->out_bf16 = dtype == UOCR_B200_BF16;
    return UOCR_B200_OK;
}

int uocr_b200_workspace_set_wait_limit(uocr_b200_workspace* ws, unsigned polls) {
    if (!ws) return fail(UOCR_B200_ERR_INVALID, "workspace_set_wait_limit: null workspace");
    ws->wait_limit = polls > kWaitLimit ? kWaitLimit : polls;
    return UOCR_B200_OK;
}

int uocr_b200_workspace_set_overlap(uocr_b200_workspace* ws, int enabled) {
    if (!ws) return fail(UOCR_B200_ERR_INVALID, "workspace_set_overlap: null workspace");
    ws->overlap = enabled != 0;
    return UOCR_B200_OK;
}

int uocr_b200_workspace_last_kernel_ms(uocr_b200_workspace* ws, float* ms) {
    if (!ws || !ms || !ws->ev0) return fail(UOCR_B200_ERR_INVALID, "workspace_last_kernel_ms: timing was never enabled");
    CHECK_CUDA(cudaEventSynchronize(ws->ev1), "event sync");
    CHECK_CUDA(cudaEventElapsedTime(ms, ws->ev0, ws->ev1), "event elapsed");
    return UOCR_B200_OK;
}

int uocr_b200_workspace_status(uocr_b200_workspace* ws, uocr_b200_stream_t stream, int* device_status) {
    if (!ws || !device_status) return fail(UOCR_B200_ERR_INVALID, "workspace_status: null argument");
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    int v = 0;
    CHECK_CUDA(cudaMemcpyAsync(&v, ws->status, sizeof(int), cudaMemcpyDeviceToHost, st), "status D2H");
    CHECK_CUDA(cudaMemsetAsync(ws->status, 0, sizeof(int), st), "status clear");
    CHECK_CUDA(cudaStreamSynchronize(st), "status sync");
    if (v != 0 && ws->counters) {
        // a kernel that gave up may have left arrival counters half-way: start clean again
        CHECK_CUDA(cudaMemsetAsync(ws->counters, 0, sizeof(int) * ((size_t)ws->pieces_max + 64), st), "counter clear");
        CHECK_CUDA(cudaStreamSynchronize(st), "counter clear sync");
    }
    *device_status = v;
    return UOCR_B200_OK;
}

}  // extern "C"

// =================================================================================================
// attention dispatch
// =================================================================================================
namespace {

struct AttnCall {
    // layout
    bool paged = false;
    int dtype = UOCR_B200_F32;
    const void* k_base = nullptr;
    const void* v_base = nullptr;
    const int32_t* table = nullptr;
    int table_stride = 0, num_blocks = 0;
    int slot_rows = 0;
    // geometry
    int rows = 0, heads = 0, kv_heads = 0, head_dim = 0;
    const float* q = nullptr;
    float* out = nullptr;
    PlanParams plan{};
    // fused decode step (append + attention in one launch)
    const void* k_text = nullptr;
    const void* v_text = nullptr;
    int text_blocks = 0;
    bool fused = false;
    const float* k_new = nullptr;
    const float* v_new = nullptr;
    int* d_len_rw = nullptr;
    int* d_ring_rw = nullptr;
    const int* rope_pos = nullptr;  // fused step with rotary embedding
    float rope_theta = 0.f;
};

// Share the last CTA of an overlapped launch gives up, in sixteenths: it starts 8-12 us after the others
// (of a launch of ~50 us), and 3/16 measured best among 0..6.
constexpr int kLateCtaSixteenths = 3;

constexpr int kFusedMaxRows = 1024;  // the fused step plans in shared memory

template <typename KV, int HD, bool PAGED, bool FUSED, bool ROPE = false>
int launch_partial(const AttnParams& ap, const DeviceInfo& di, int* warps_used, cudaStream_t st, bool dry,
                   bool overlap = false) {
    using M = TileMap<KV, HD>;
    constexpr int per_warp = kRing * M::kTileBytes;
    const int plan_bytes = FUSED ? (int)(sizeof(RowInfo) * ap.rows + sizeof(int) * (3 * ap.rows + 1 + 33) + 128) : 0;
    const int budget = (di.smem_optin < 200 * 1024 ? di.smem_optin : 200 * 1024) - 1024 - plan_bytes -
                       kMaxWarpsPerCta * kPendMax * (int)sizeof(int);
    int warps = budget / per_warp;
    if (warps > kMaxWarpsPerCta) warps = kMaxWarpsPerCta;
    if (warps < 1) return fail(UOCR_B200_ERR_UNSUPPORTED, "tile does not fit in shared memory");
    constexpr int ctas = 1;  // one persistent CTA per SM
    *warps_used = warps;
    if (dry) return UOCR_B200_OK;
    const int bar_bytes = (warps * kRing * 8 + 127) & ~127;
    const int smem = bar_bytes + warps * per_warp + warps * kPendMax * (int)sizeof(int) + plan_bytes;
    auto kern = rswa_attn_kernel<KV, HD, PAGED, FUSED, ROPE>;
    static int configured_smem[64] = {0};  // one per instantiation of this template
    int dev = 0;
    cudaGetDevice(&dev);
    if (configured_smem[dev] < smem) {
        CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem), "smem attribute");
        configured_smem[dev] = smem;
    }
    if (FUSED && overlap) {
        // programmatic dependent launch: this grid may become resident while the previous kernel in the
        // stream is still draining; the kernel itself waits for it before consuming inputs or scratch
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(di.sms * ctas);
        cfg.blockDim = dim3(warps * 32);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = st;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        CHECK_CUDA(cudaLaunchKernelEx(&cfg, kern, ap), "attention kernel launch");
    } else {
        kern<<<di.sms * ctas, warps * 32, smem, st>>>(ap);
    }
    return after_launch("attention kernel");
}

template <typename KV, bool PAGED, bool FUSED, bool ROPE = false>
int dispatch_hd(int hd, const AttnParams& ap, const DeviceInfo& di, int* warps, cudaStream_t st, bool dry, bool ov) {
    switch (hd) {
        case 8:
            if constexpr (!ROPE || KV::kBytes == 4) return launch_partial<KV, 8, PAGED, FUSED, ROPE>(ap, di, warps, st, dry, ov);
            break;
        case 16: return launch_partial<KV, 16, PAGED, FUSED, ROPE>(ap, di, warps, st, dry, ov);
        case 32: return launch_partial<KV, 32, PAGED, FUSED, ROPE>(ap, di, warps, st, dry, ov);
        case 64: return launch_partial<KV, 64, PAGED, FUSED, ROPE>(ap, di, warps, st, dry, ov);
        case 128: return launch_partial<KV, 128, PAGED, FUSED, ROPE>(ap, di, warps, st, dry, ov);
        case 256: return launch_partial<KV, 256, PAGED, FUSED, ROPE>(ap, di, warps, st, dry, ov);
        case 4:
            if constexpr (KV::kBytes == 4 && !ROPE) return launch_partial<KV, 4, PAGED, FUSED, ROPE>(ap, di, warps, st, dry, ov);
            break;
        default: break;
    }
    if (ROPE) return fail(UOCR_B200_ERR_UNSUPPORTED, "rotary step: head_dim must be a power of two in [16,256] (bf16) or [8,256] (fp32)");
    return fail(UOCR_B200_ERR_UNSUPPORTED, "head_dim must be a power of two in [8,256] (bf16) or [4,256] (fp32)");
}

int dispatch_partial(const AttnCall& c, const AttnParams& ap, const DeviceInfo& di, int* warps, cudaStream_t st, bool dry, bool ov = false) {
    if (c.fused && c.rope_pos) {
        if (c.dtype == UOCR_B200_BF16) return dispatch_hd<BF16, true, true, true>(c.head_dim, ap, di, warps, st, dry, ov);
        return dispatch_hd<F32, true, true, true>(c.head_dim, ap, di, warps, st, dry, ov);
    }
    if (c.fused) {
        if (c.dtype == UOCR_B200_BF16) return dispatch_hd<BF16, true, true>(c.head_dim, ap, di, warps, st, dry, ov);
        return dispatch_hd<F32, true, true>(c.head_dim, ap, di, warps, st, dry, ov);
    }
    if (c.paged) {
        if (c.dtype == UOCR_B200_BF16) return dispatch_hd<BF16, true, false>(c.head_dim, ap, di, warps, st, dry, ov);
        return dispatch_hd<F32, true, false>(c.head_dim, ap, di, warps, st, dry, ov);
    }
    return dispatch_hd<F32, false, false>(c.head_dim, ap, di, warps, st, dry, ov);
}

int run_attention(AttnCall& c, uocr_b200_workspace* ws, cudaStream_t st) {
    if (c.rows <= 0) return UOCR_B200_OK;  // the reference wrappers return early on empty batches
    if (!ws) return fail(UOCR_B200_ERR_INVALID, "attention: workspace is null");
    if (!c.q || !c.out || !c.k_base || !c.v_base) return fail(UOCR_B200_ERR_INVALID, "attention: null pointer");
    if (c.heads <= 0 || c.kv_heads <= 0 || c.heads % c.kv_heads != 0)
        return fail(UOCR_B200_ERR_INVALID, "attention: heads must be a positive multiple of kv_heads");
    if (!head_dim_ok(c.head_dim, c.dtype)) return fail(UOCR_B200_ERR_UNSUPPORTED, "attention: unsupported head_dim");
    if (!aligned16(c.q) || !aligned16(c.out) || !aligned16(c.k_base) || !aligned16(c.v_base))
        return fail(UOCR_B200_ERR_INVALID, "attention: q/out/cache pointers must be 16-byte aligned");
    if (c.rows > ws->max_rows) return fail(UOCR_B200_ERR_WORKSPACE, "attention: more rows than the workspace was created for");
    const DeviceInfo* di = nullptr;
    if (int rc = device_info(&di)) return rc;

    AttnParams ap{};
    ap.q = c.q;
    ap.out = c.out;
    ap.out_bf16 = ws->out_bf16 ? 1 : 0;
    ap.k_base = static_cast<const uint8_t*>(c.k_base);
    ap.v_base = static_cast<const uint8_t*>(c.v_base);
    ap.k_text = static_cast<const uint8_t*>(c.k_text);
    ap.v_text = static_cast<const uint8_t*>(c.v_text);
    ap.text_blocks = c.text_blocks;
    ap.table = c.table;
    ap.table_stride = c.table_stride;
    ap.num_blocks = c.num_blocks;
    ap.slot_rows = c.slot_rows;
    ap.row_stride_bytes = c.kv_heads * c.head_dim * 4;
    ap.rows = c.rows;
    ap.heads = c.heads;
    ap.kv_heads = c.kv_heads;
    ap.group = c.heads / c.kv_heads;
    ap.scale_log2e = (1.0f / std::sqrt(static_cast<float>(c.head_dim))) * 1.4426950408889634f;
    ap.rs = ws->rs;
    ap.info = ws->info;
    ap.part_acc = ws->part_acc;
    ap.part_ml = ws->part_ml;
    ap.counters = ws->counters;
    ap.status = ws->status;
    ap.k_new = c.k_new;
    ap.v_new = c.v_new;
    ap.d_len = c.d_len_rw;
    ap.d_ring_pos = c.d_ring_rw;
    ap.planned_ctas = ws->planned_ctas;
    ap.late_cta = (c.fused && ws->overlap) ? kLateCtaSixteenths : 0;
    ap.wait_limit = ws->wait_limit;
    if (c.rope_pos) {
        ap.rope_pos = c.rope_pos;
        // same float expression as the reference (src/kernels/cpu_ops.cpp:163; rope_fused.cu:22)
        for (int i = 0; i < c.head_dim / 2; ++i) ap.rope_freq[i] = std::pow(c.rope_theta, -2.0f * i / static_cast<float>(c.head_dim));
    }

    c.plan.rows = c.rows;
    c.plan.heads = c.heads;
    c.plan.paged = c.paged ? 1 : 0;
    c.plan.rs = ws->rs;
    c.plan.info = ws->info;
    c.plan.out = c.fused ? nullptr : c.out;
    c.plan.out_row_elems = c.heads * c.head_dim / (ws->out_bf16 ? 2 : 1);  // zero-filled as 32-bit words
    ap.plan = c.plan;

    int warps = 0;
    if (int rc = dispatch_partial(c, ap, *di, &warps, st, /*dry=*/true)) return rc;
    ap.total_warps = di->sms * warps;
    if (ap.total_warps > ws->total_warps_max) return fail(UOCR_B200_ERR_WORKSPACE, "attention: workspace built for a smaller device");

    if (!c.fused) {
        int pthreads = c.rows < 1024 ? ((c.rows + 31) & ~31) : 1024;
        rswa_plan_kernel<<<1, pthreads, 0, st>>>(c.plan);
        if (int rc = after_launch("plan kernel")) return rc;
    }
    if (ws->timing) CHECK_CUDA(cudaEventRecord(ws->ev0, st), "event record");
    if (int rc = dispatch_partial(c, ap, *di, &warps, st, /*dry=*/false, ws->overlap)) return rc;
    if (ws->timing) CHECK_CUDA(cudaEventRecord(ws->ev1, st), "event record");
    return UOCR_B200_OK;
}

int fill_paged(AttnCall& c, const uocr_b200_paged_kv* kv) {
    if (!kv) return fail(UOCR_B200_ERR_INVALID, "paged view is null");
    if (kv->dtype != UOCR_B200_BF16 && kv->dtype != UOCR_B200_F32) return fail(UOCR_B200_ERR_UNSUPPORTED, "paged dtype must be bf16 or fp32");
    if (!kv->block_table || kv->table_stride <= 0 || kv->num_blocks <= 0) return fail(UOCR_B200_ERR_INVALID, "paged view: bad block table");
    c.paged = true;
    c.dtype = kv->dtype;
    c.k_base = kv->k_pool;
    c.v_base = kv->v_pool;
    c.table = kv->block_table;
    c.table_stride = kv->table_stride;
    c.num_blocks = kv->num_blocks;
    c.kv_heads = kv->kv_heads;
    c.head_dim = kv->head_dim;
    return UOCR_B200_OK;
}

int paged_view(const uocr_b200_paged_kv* kv, PagedView* pv) {
    if (!kv || !kv->k_pool || !kv->v_pool || !kv->block_table) return fail(UOCR_B200_ERR_INVALID, "paged view: null pointer");
    if (kv->dtype != UOCR_B200_BF16 && kv->dtype != UOCR_B200_F32) return fail(UOCR_B200_ERR_UNSUPPORTED, "paged dtype must be bf16 or fp32");
    if (!head_dim_ok(kv->head_dim, kv->dtype) || kv->kv_heads <= 0) return fail(UOCR_B200_ERR_UNSUPPORTED, "paged view: unsupported head geometry");
    if (!aligned16(kv->k_pool) || !aligned16(kv->v_pool)) return fail(UOCR_B200_ERR_INVALID, "paged view: pools must be 16-byte aligned");
    pv->k_pool = static_cast<uint8_t*>(kv->k_pool);
    pv->v_pool = static_cast<uint8_t*>(kv->v_pool);
    pv->table = kv->block_table;
    pv->table_stride = kv->table_stride;
    pv->num_blocks = kv->num_blocks;
    pv->kv_heads = kv->kv_heads;
    pv->head_dim = kv->head_dim;
    return UOCR_B200_OK;
}

}  // namespace

extern "C" {

// ---- append ---------------------------------------------------------------------------------------
int uocr_b200_rswa_append_decode_batch_f32(const float* k, const float* v, float* kbase, float* vbase,
                                           int* d_len, int* d_ring_pos, const int* d_prefill_len,
                                           const int* d_slots, int batch, int batch_cap, int window,
                                           int kv_heads, int head_dim, uocr_b200_stream_t stream) {
    if (batch <= 0) return UOCR_B200_OK;
    if (!k || !v || !kbase || !vbase || !d_len || !d_ring_pos || !d_prefill_len || !d_slots)
        return fail(UOCR_B200_ERR_INVALID, "append_decode_batch_f32: null pointer");
    if (window <= 0 || kv_heads <= 0 || head_dim <= 0 || batch_cap <= 0) return fail(UOCR_B200_ERR_INVALID, "append_decode_batch_f32: bad geometry");
    int stride = kv_heads * head_dim;
    const bool vec = (stride % 4 == 0) && aligned16(k) && aligned16(v) && aligned16(kbase) && aligned16(vbase);
    rswa_append_f32_kernel<<<batch, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        k, v, kbase, vbase, d_len, d_ring_pos, d_prefill_len, d_slots, 0, batch_cap, window,
        vec ? stride : -stride);
    return after_launch("append (fp32, batched)");
}

int uocr_b200_rswa_append_decode_f32(const float* k, const float* v, float* kcache, float* vcache,
                                     int* d_len, int* d_ring_pos, int prefill_len, int window,
                                     int kv_heads, int head_dim, uocr_b200_stream_t stream) {
    if (!k || !v || !kcache || !vcache || !d_len || !d_ring_pos) return fail(UOCR_B200_ERR_INVALID, "append_decode_f32: null pointer");
    if (window <= 0 || kv_heads <= 0 || head_dim <= 0 || prefill_len < 0) return fail(UOCR_B200_ERR_INVALID, "append_decode_f32: bad geometry");
    int stride = kv_heads * head_dim;
    const bool vec = (stride % 4 == 0) && aligned16(k) && aligned16(v) && aligned16(kcache) && aligned16(vcache);
    rswa_append_f32_kernel<<<1, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        k, v, kcache, vcache, d_len, d_ring_pos, nullptr, nullptr, prefill_len, 0, window,
        vec ? stride : -stride);
    return after_launch("append (fp32, single)");
}

int uocr_b200_rswa_append_decode_batch_paged(const uocr_b200_paged_kv* kv, const float* k, const float* v,
                                             int* d_len, int* d_ring_pos, const int* d_prefill_len,
                                             const int* d_slots, int batch, int window,
                                             uocr_b200_workspace* ws, uocr_b200_stream_t stream) {
    if (batch <= 0) return UOCR_B200_OK;
    PagedView pv;
    if (int rc = paged_view(kv, &pv)) return rc;
    if (!k || !v || !d_len || !d_ring_pos || !d_prefill_len || !d_slots) return fail(UOCR_B200_ERR_INVALID, "append_decode_batch_paged: null pointer");
    if (!aligned16(k) || !aligned16(v)) return fail(UOCR_B200_ERR_INVALID, "append_decode_batch_paged: k/v must be 16-byte aligned");
    if (window <= 0) return fail(UOCR_B200_ERR_INVALID, "append_decode_batch_paged: window must be positive");
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    int* status = ws ? ws->status : nullptr;
    if (kv->dtype == UOCR_B200_BF16)
        rswa_append_paged_kernel<BF16><<<batch, 256, 0, st>>>(pv, k, v, d_len, d_ring_pos, d_prefill_len, d_slots, window, status);
    else
        rswa_append_paged_kernel<F32><<<batch, 256, 0, st>>>(pv, k, v, d_len, d_ring_pos, d_prefill_len, d_slots, window, status);
    return after_launch("append (paged)");
}

// Checks that `layers` views describe pools of one geometry behind one block table and collects the pools.
static int collect_layers(const uocr_b200_paged_kv* kv, int layers, PagedView* pv, LayerPools* pools, const char* who) {
    if (!kv || layers <= 0 || layers > kMaxLayersPerLaunch)
        return fail(UOCR_B200_ERR_INVALID, std::string(who) + ": 1..32 layers per call");
    if (int rc = paged_view(&kv[0], pv)) return rc;
    for (int l = 0; l < layers; ++l) {
        PagedView one;
        if (int rc = paged_view(&kv[l], &one)) return rc;
        if (kv[l].dtype != kv[0].dtype || one.table != pv->table || one.table_stride != pv->table_stride ||
            one.num_blocks != pv->num_blocks || one.kv_heads != pv->kv_heads || one.head_dim != pv->head_dim)
            return fail(UOCR_B200_ERR_INVALID, std::string(who) + ": the layers must share block table, geometry and dtype");
        pools->k[l] = one.k_pool;
        pools->v[l] = one.v_pool;
    }
    return UOCR_B200_OK;
}

int uocr_b200_rswa_append_decode_batch_paged_layers(const uocr_b200_paged_kv* kv_layers, int layers, const float* k,
                                                    const float* v, long long kv_layer_stride, int* d_len, int* d_ring_pos,
                                                    long long cursor_layer_stride, const int* d_prefill_len,
                                                    const int* d_slots, int batch, int window, uocr_b200_workspace* ws,
                                                    uocr_b200_stream_t stream) {
    if (batch <= 0) return UOCR_B200_OK;
    PagedView pv;
    LayerPools pools{};
    if (int rc = collect_layers(kv_layers, layers, &pv, &pools, "append_decode_batch_paged_layers")) return rc;
    if (!k || !v || !d_len || !d_ring_pos || !d_prefill_len || !d_slots) return fail(UOCR_B200_ERR_INVALID, "append_decode_batch_paged_layers: null pointer");
    if (!aligned16(k) || !aligned16(v) || (kv_layer_stride & 3)) return fail(UOCR_B200_ERR_INVALID, "append_decode_batch_paged_layers: k/v and the layer stride must be 16-byte aligned");
    if (window <= 0) return fail(UOCR_B200_ERR_INVALID, "append_decode_batch_paged_layers: window must be positive");
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    int* status = ws ? ws->status : nullptr;
    const dim3 grid(batch, 1, layers);
    if (kv_layers[0].dtype == UOCR_B200_BF16)
        rswa_append_paged_layers_kernel<BF16><<<grid, 256, 0, st>>>(pv, pools, k, v, kv_layer_stride, d_len, d_ring_pos, cursor_layer_stride, d_prefill_len, d_slots, window, status);
    else
        rswa_append_paged_layers_kernel<F32><<<grid, 256, 0, st>>>(pv, pools, k, v, kv_layer_stride, d_len, d_ring_pos, cursor_layer_stride, d_prefill_len, d_slots, window, status);
    return after_launch("append (paged, all layers)");
}

int uocr_b200_rswa_gather_paged_layers(const uocr_b200_paged_kv* kv_layers, int layers, const int* d_len,
                                       long long cursor_layer_stride, const int* d_prefill_len, const int* d_slots, int n,
                                       int capacity_rows, void* out_k, void* out_v, long long out_layer_stride_bytes,
                                       int out_dtype, uocr_b200_workspace* ws, uocr_b200_stream_t stream) {
    if (n <= 0 || capacity_rows <= 0) return UOCR_B200_OK;
    PagedView pv;
    LayerPools pools{};
    if (int rc = collect_layers(kv_layers, layers, &pv, &pools, "gather_paged_layers")) return rc;
    if (!d_len || !d_prefill_len || !d_slots || !out_k || !out_v) return fail(UOCR_B200_ERR_INVALID, "gather_paged_layers: null pointer");
    if (!aligned16(out_k) || !aligned16(out_v) || (out_layer_stride_bytes & 15)) return fail(UOCR_B200_ERR_INVALID, "gather_paged_layers: outputs and the layer stride must be 16-byte aligned");
    const int dtype = kv_layers[0].dtype;
    if (out_dtype != UOCR_B200_F32 && out_dtype != dtype) return fail(UOCR_B200_ERR_UNSUPPORTED, "gather_paged_layers: out_dtype must be fp32 or the pool dtype");
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    int* status = ws ? ws->status : nullptr;
    const dim3 grid(capacity_rows, n, layers);
    uint8_t* ok = static_cast<uint8_t*>(out_k);
    uint8_t* ov = static_cast<uint8_t*>(out_v);
    if (dtype == UOCR_B200_BF16 && out_dtype == UOCR_B200_F32)
        rswa_gather_paged_layers_kernel<BF16, true><<<grid, 160, 0, st>>>(pv, pools, d_len, cursor_layer_stride, d_prefill_len, d_slots, capacity_rows, ok, ov, out_layer_stride_bytes, status);
    else if (dtype == UOCR_B200_BF16)
        rswa_gather_paged_layers_kernel<BF16, false><<<grid, 160, 0, st>>>(pv, pools, d_len, cursor_layer_stride, d_prefill_len, d_slots, capacity_rows, ok, ov, out_layer_stride_bytes, status);
    else
        rswa_gather_paged_layers_kernel<F32, false><<<grid, 160, 0, st>>>(pv, pools, d_len, cursor_layer_stride, d_prefill_len, d_slots, capacity_rows, ok, ov, out_layer_stride_bytes, status);
    return after_launch("gather (paged, all layers)");
}

// ---- prefill scatter --------------------------------------------------------------------------------
int uocr_b200_rswa_write_prefill_ragged_f32(const float* k, const float* v, float* kbase, float* vbase,
                                            const int* d_slots, const int* d_pos, int total, int batch_cap,
                                            int kv_heads, int head_dim, uocr_b200_stream_t stream) {
    if (total <= 0) return UOCR_B200_OK;
    if (!k || !v || !kbase || !vbase || !d_slots || !d_pos) return fail(UOCR_B200_ERR_INVALID, "write_prefill_ragged_f32: null pointer");
    if (kv_heads <= 0 || head_dim <= 0 || batch_cap <= 0) return fail(UOCR_B200_ERR_INVALID, "write_prefill_ragged_f32: bad geometry");
    int stride = kv_heads * head_dim;
    const bool vec = (stride % 4 == 0) && aligned16(k) && aligned16(v) && aligned16(kbase) && aligned16(vbase);
    rswa_scatter_f32_kernel<<<total, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        k, v, kbase, vbase, d_slots, d_pos, batch_cap, vec ? stride : -stride);
    return after_launch("prefill scatter (fp32)");
}

int uocr_b200_rswa_write_prefill_ragged_paged(const uocr_b200_paged_kv* kv, const float* k, const float* v,
                                              const int* d_slots, const int* d_pos, int total,
                                              uocr_b200_workspace* ws, uocr_b200_stream_t stream) {
    if (total <= 0) return UOCR_B200_OK;
    PagedView pv;
    if (int rc = paged_view(kv, &pv)) return rc;
    if (!k || !v || !d_slots || !d_pos) return fail(UOCR_B200_ERR_INVALID, "write_prefill_ragged_paged: null pointer");
    if (!aligned16(k) || !aligned16(v)) return fail(UOCR_B200_ERR_INVALID, "write_prefill_ragged_paged: k/v must be 16-byte aligned");
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    int* status = ws ? ws->status : nullptr;
    if (kv->dtype == UOCR_B200_BF16)
        rswa_scatter_paged_kernel<BF16><<<total, 256, 0, st>>>(pv, k, v, d_slots, d_pos, status);
    else
        rswa_scatter_paged_kernel<F32><<<total, 256, 0, st>>>(pv, k, v, d_slots, d_pos, status);
    return after_launch("prefill scatter (paged)");
}

// ---- slot state publication ---------------------------------------------------------------------------
int uocr_b200_rswa_publish_slots(const int32_t* d_packed, int n, int32_t* block_table, int table_stride, int* d_len,
                                 int* d_ring_pos, int* d_prefill_len, int slots, int layers, uocr_b200_workspace* ws,
                                 uocr_b200_stream_t stream) {
    if (n <= 0) return UOCR_B200_OK;
    if (!d_packed || !block_table || !d_len || !d_ring_pos || !d_prefill_len) return fail(UOCR_B200_ERR_INVALID, "publish_slots: null pointer");
    if (table_stride <= 0 || slots <= 0 || layers <= 0) return fail(UOCR_B200_ERR_INVALID, "publish_slots: bad geometry");
    rswa_publish_slots_kernel<<<n, 128, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        d_packed, block_table, table_stride, d_len, d_ring_pos, d_prefill_len, slots, layers, ws ? ws->status : nullptr);
    return after_launch("slot state publication");
}

// ---- attention ----------------------------------------------------------------------------------------
int uocr_b200_rswa_attention_batch_f32(const float* q, const float* kbase, const float* vbase, const int* d_len,
                                       const int* d_slots, int batch, int batch_cap, int heads, int kv_heads,
                                       int head_dim, float* out, uocr_b200_workspace* ws, uocr_b200_stream_t stream) {
    if (batch <= 0) return UOCR_B200_OK;
    if (!d_len || !d_slots) return fail(UOCR_B200_ERR_INVALID, "attention_batch_f32: null index array");
    AttnCall c;
    c.k_base = kbase; c.v_base = vbase;
    c.slot_rows = batch_cap;
    c.rows = batch; c.heads = heads; c.kv_heads = kv_heads; c.head_dim = head_dim;
    c.q = q; c.out = out;
    c.plan.mode = kPlanBatch; c.plan.d_slots = d_slots; c.plan.d_len = d_len;
    return run_attention(c, ws, reinterpret_cast<cudaStream_t>(stream));
}

int uocr_b200_rswa_attention_batch_paged(const uocr_b200_paged_kv* kv, const float* q, const int* d_len,
                                         const int* d_prefill_len, const int* d_slots, int batch, int heads,
                                         float* out, uocr_b200_workspace* ws, uocr_b200_stream_t stream) {
    if (batch <= 0) return UOCR_B200_OK;
    if (!d_len || !d_slots || !d_prefill_len) return fail(UOCR_B200_ERR_INVALID, "attention_batch_paged: null index array");
    AttnCall c;
    if (int rc = fill_paged(c, kv)) return rc;
    c.rows = batch; c.heads = heads; c.q = q; c.out = out;
    c.plan.mode = kPlanBatch; c.plan.d_slots = d_slots; c.plan.d_len = d_len; c.plan.d_prefill_len = d_prefill_len;
    return run_attention(c, ws, reinterpret_cast<cudaStream_t>(stream));
}

int uocr_b200_rswa_attention_ragged_f32(const float* q, const float* kbase, const float* vbase, const int* d_slots,
                                        const int* d_pos, int total, int batch_cap, int heads, int kv_heads,
                                        int head_dim, float* out, uocr_b200_workspace* ws, uocr_b200_stream_t stream) {
    if (total <= 0) return UOCR_B200_OK;
    if (!d_slots || !d_pos) return fail(UOCR_B200_ERR_INVALID, "attention_ragged_f32: null index array");
    AttnCall c;
    c.k_base = kbase; c.v_base = vbase;
    c.slot_rows = batch_cap;
    c.rows = total; c.heads = heads; c.kv_heads = kv_heads; c.head_dim = head_dim;
    c.q = q; c.out = out;
    c.plan.mode = kPlanRagged; c.plan.d_slots = d_slots; c.plan.d_pos = d_pos;
    return run_attention(c, ws, reinterpret_cast<cudaStream_t>(stream));
}

int uocr_b200_rswa_attention_ragged_paged(const uocr_b200_paged_kv* kv, const float* q, const int* d_prefill_len,
                                          const int* d_slots, const int* d_pos, int total, int heads, float* out,
                                          uocr_b200_workspace* ws, uocr_b200_stream_t stream) {
    if (total <= 0) return UOCR_B200_OK;
    if (!d_slots || !d_pos || !d_prefill_len) return fail(UOCR_B200_ERR_INVALID, "attention_ragged_paged: null index array");
    AttnCall c;
    if (int rc = fill_paged(c, kv)) return rc;
    c.rows = total; c.heads = heads; c.q = q; c.out = out;
    c.plan.mode = kPlanRagged; c.plan.d_slots = d_slots; c.plan.d_pos = d_pos; c.plan.d_prefill_len = d_prefill_len;
    return run_attention(c, ws, reinterpret_cast<cudaStream_t>(stream));
}

int uocr_b200_rswa_attention_f32(const float* q, const float* kcache, const float* vcache, int kv_len, const int* d_len,
                                 int seq, int q_start, int heads, int kv_heads, int head_dim, int causal, float* out,
                                 uocr_b200_workspace* ws, uocr_b200_stream_t stream) {
    if (seq <= 0) return UOCR_B200_OK;
    AttnCall c;
    c.k_base = kcache; c.v_base = vcache;
    c.slot_rows = 0;
    c.rows = seq; c.heads = heads; c.kv_heads = kv_heads; c.head_dim = head_dim;
    c.q = q; c.out = out;
    c.plan.mode = kPlanSingle; c.plan.fixed_slot = 0; c.plan.kv_len = kv_len; c.plan.d_len = d_len;
    c.plan.q_start = q_start; c.plan.causal = causal ? 1 : 0;
    return run_attention(c, ws, reinterpret_cast<cudaStream_t>(stream));
}

int uocr_b200_rswa_attention_paged(const uocr_b200_paged_kv* kv, int slot, const float* q, int kv_len, const int* d_len,
                                   int prefill_len, const int* d_prefill_len, int seq, int q_start, int heads, int causal,
                                   float* out, uocr_b200_workspace* ws, uocr_b200_stream_t stream) {
    if (seq <= 0) return UOCR_B200_OK;
    if (slot < 0) return fail(UOCR_B200_ERR_INVALID, "attention_paged: negative slot");
    AttnCall c;
    if (int rc = fill_paged(c, kv)) return rc;
    c.rows = seq; c.heads = heads; c.q = q; c.out = out;
    c.plan.mode = kPlanSingle; c.plan.fixed_slot = slot; c.plan.kv_len = kv_len; c.plan.d_len = d_len;
    c.plan.prefill_len = prefill_len; c.plan.d_prefill_len = d_prefill_len;
    c.plan.q_start = q_start; c.plan.causal = causal ? 1 : 0;
    return run_attention(c, ws, reinterpret_cast<cudaStream_t>(stream));
}

// ---- text prefill over prefix + window ----------------------------------------------------------------
int uocr_b200_rswa_prefill_text_paged(const uocr_b200_paged_kv* kv, void* text_k_pool, void* text_v_pool, int text_blocks,
                                      const float* q, const float* k, const float* v, const int* d_prefill_len,
                                      const int* d_slots, const int* d_pos, const int* d_text_block0, int total,
                                      int window, int heads, float* out, uocr_b200_workspace* ws,
                                      uocr_b200_stream_t stream) {
    if (total <= 0) return UOCR_B200_OK;
    PagedView pv;
    if (int rc = paged_view(kv, &pv)) return rc;
    if (!text_k_pool || !text_v_pool || text_blocks <= 0 || !k || !v || !d_prefill_len || !d_slots || !d_pos || !d_text_block0)
        return fail(UOCR_B200_ERR_INVALID, "prefill_text_paged: null pointer");
    if (!aligned16(text_k_pool) || !aligned16(text_v_pool) || !aligned16(k) || !aligned16(v))
        return fail(UOCR_B200_ERR_INVALID, "prefill_text_paged: pointers must be 16-byte aligned");
    if (window <= 0) return fail(UOCR_B200_ERR_INVALID, "prefill_text_paged: window must be positive");
    if (!ws) return fail(UOCR_B200_ERR_INVALID, "prefill_text_paged: workspace is null");
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    PagedView text = pv;
    text.k_pool = static_cast<uint8_t*>(text_k_pool);
    text.v_pool = static_cast<uint8_t*>(text_v_pool);
    text.table = nullptr;
    text.table_stride = 0;
    text.num_blocks = text_blocks;
    if (kv->dtype == UOCR_B200_BF16)
        rswa_scatter_text_kernel<BF16><<<total, 256, 0, st>>>(text, k, v, d_pos, d_text_block0, ws->status);
    else
        rswa_scatter_text_kernel<F32><<<total, 256, 0, st>>>(text, k, v, d_pos, d_text_block0, ws->status);
    if (int rc = after_launch("text scatter")) return rc;
    AttnCall c;
    if (int rc = fill_paged(c, kv)) return rc;
    c.k_text = text_k_pool; c.v_text = text_v_pool; c.text_blocks = text_blocks;
    c.rows = total; c.heads = heads; c.q = q; c.out = out;
    c.plan.mode = kPlanPrefillText; c.plan.d_slots = d_slots; c.plan.d_pos = d_pos; c.plan.d_prefill_len = d_prefill_len;
    c.plan.d_text_block0 = d_text_block0; c.plan.window = window;
    return run_attention(c, ws, st);
}

int uocr_b200_rswa_ring_fill_paged(const uocr_b200_paged_kv* kv, const void* text_k_pool, const void* text_v_pool,
                                   int text_blocks, const int* d_slots, const int* d_pos, const int* d_text_block0,
                                   const int* d_text_len, const int* d_prefill_len, int* d_len, int* d_ring_pos,
                                   int total, int window, uocr_b200_workspace* ws, uocr_b200_stream_t stream) {
    if (total <= 0) return UOCR_B200_OK;
    PagedView pv;
    if (int rc = paged_view(kv, &pv)) return rc;
    if (!text_k_pool || !text_v_pool || text_blocks <= 0 || !d_slots || !d_pos || !d_text_block0 || !d_text_len ||
        !d_prefill_len || !d_len || !d_ring_pos)
        return fail(UOCR_B200_ERR_INVALID, "ring_fill_paged: null pointer");
    if (window <= 0) return fail(UOCR_B200_ERR_INVALID, "ring_fill_paged: window must be positive");
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    int* status = ws ? ws->status : nullptr;
    const uint8_t* kt = static_cast<const uint8_t*>(text_k_pool);
    const uint8_t* vt = static_cast<const uint8_t*>(text_v_pool);
    if (kv->dtype == UOCR_B200_BF16)
        rswa_ring_fill_kernel<BF16><<<total, 160, 0, st>>>(pv, kt, vt, d_slots, d_pos, d_text_block0, d_text_len, d_prefill_len, d_len, d_ring_pos, window, status);
    else
        rswa_ring_fill_kernel<F32><<<total, 160, 0, st>>>(pv, kt, vt, d_slots, d_pos, d_text_block0, d_text_len, d_prefill_len, d_len, d_ring_pos, window, status);
    return after_launch("ring fill");
}

int uocr_b200_rswa_text_scatter_paged(const uocr_b200_paged_kv* kv, void* text_k_pool, void* text_v_pool, int text_blocks,
                                      const float* k, const float* v, const int* d_pos, const int* d_text_block0,
                                      int total, uocr_b200_workspace* ws, uocr_b200_stream_t stream) {
    if (total <= 0) return UOCR_B200_OK;
    PagedView pv;
    if (int rc = paged_view(kv, &pv)) return rc;
    if (!text_k_pool || !text_v_pool || text_blocks <= 0 || !k || !v || !d_pos || !d_text_block0)
        return fail(UOCR_B200_ERR_INVALID, "text_scatter_paged: null pointer");
    if (!aligned16(text_k_pool) || !aligned16(text_v_pool) || !aligned16(k) || !aligned16(v))
        return fail(UOCR_B200_ERR_INVALID, "text_scatter_paged: pointers must be 16-byte aligned");
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    PagedView text = pv;
    text.k_pool = static_cast<uint8_t*>(text_k_pool);
    text.v_pool = static_cast<uint8_t*>(text_v_pool);
    text.table = nullptr;
    text.table_stride = 0;
    text.num_blocks = text_blocks;
    int* status = ws ? ws->status : nullptr;
    if (kv->dtype == UOCR_B200_BF16)
        rswa_scatter_text_kernel<BF16><<<total, 256, 0, st>>>(text, k, v, d_pos, d_text_block0, status);
    else
        rswa_scatter_text_kernel<F32><<<total, 256, 0, st>>>(text, k, v, d_pos, d_text_block0, status);
    return after_launch("text scatter");
}

int uocr_b200_rswa_text_scatter_fill_paged(const uocr_b200_paged_kv* kv, void* text_k_pool, void* text_v_pool, int text_blocks,
                                           const float* k, const float* v, const int* d_slots, const int* d_pos,
                                           const int* d_text_block0, const int* d_text_len, const int* d_prefill_len,
                                           int* d_len, int* d_ring_pos, int total, int window, uocr_b200_workspace* ws,
                                           uocr_b200_stream_t stream) {
    if (total <= 0) return UOCR_B200_OK;
    PagedView pv;
    if (int rc = paged_view(kv, &pv)) return rc;
    if (!text_k_pool || !text_v_pool || text_blocks <= 0 || !k || !v || !d_slots || !d_pos || !d_text_block0 || !d_text_len ||
        !d_prefill_len || !d_len || !d_ring_pos)
        return fail(UOCR_B200_ERR_INVALID, "text_scatter_fill_paged: null pointer");
    if (!aligned16(text_k_pool) || !aligned16(text_v_pool) || !aligned16(k) || !aligned16(v))
        return fail(UOCR_B200_ERR_INVALID, "text_scatter_fill_paged: pointers must be 16-byte aligned");
    if (window <= 0) return fail(UOCR_B200_ERR_INVALID, "text_scatter_fill_paged: window must be positive");
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    PagedView text = pv;
    text.k_pool = static_cast<uint8_t*>(text_k_pool);
    text.v_pool = static_cast<uint8_t*>(text_v_pool);
    text.table = nullptr;
    text.table_stride = 0;
    text.num_blocks = text_blocks;
    int* status = ws ? ws->status : nullptr;
    if (kv->dtype == UOCR_B200_BF16)
        rswa_scatter_text_fill_kernel<BF16><<<total, 160, 0, st>>>(pv, text, k, v, d_slots, d_pos, d_text_block0, d_text_len,
                                                                   d_prefill_len, d_len, d_ring_pos, window, status);
    else
        rswa_scatter_text_fill_kernel<F32><<<total, 160, 0, st>>>(pv, text, k, v, d_slots, d_pos, d_text_block0, d_text_len,
                                                                  d_prefill_len, d_len, d_ring_pos, window, status);
    return after_launch("text scatter + ring fill");
}

// Tensor map of a K or V pool seen as a [rows][128] bf16 matrix, fetched in boxes of 16 rows x 64
// elements (one 16-token block of one head, one 128-byte half of each row) with the 128-byte swizzle
// the tensor-core operand layout uses.  Rows at or beyond `rows` read as zeros.
static int make_kv_map(CUtensorMap* map, const void* pool, long rows) {
    using EncodeTiled = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                     const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                     CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static EncodeTiled encode = [] {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult found;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &found) != cudaSuccess ||
            found != cudaDriverEntryPointSuccess)
            fn = nullptr;
        return reinterpret_cast<EncodeTiled>(fn);
    }();
    if (!encode) return fail(UOCR_B200_ERR_CUDA, "prefill_attention_tc: the driver does not export the tensor-map encoder");
    if (!aligned16(pool) || rows <= 0 || rows >= (1L << 31))
        return fail(UOCR_B200_ERR_INVALID, "prefill_attention_tc: pool must be 16-byte aligned and hold fewer than 2^31 token rows");
    const cuuint64_t dims[2] = {(cuuint64_t)kTcTile, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)kTcTile * 2};
    const cuuint32_t box[2] = {64, (cuuint32_t)kBlockTokens};
    const cuuint32_t elem_strides[2] = {1, 1};
    const CUresult rc = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(pool), dims, strides, box, elem_strides,
                               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) return fail(UOCR_B200_ERR_CUDA, "prefill_attention_tc: tensor-map encoding failed");
    return UOCR_B200_OK;
}

// Uploads the tile descriptors and orders them on the device (the prefix lengths live there).
static int prefill_plan(const uocr_b200_prefill_tile* h_tiles, int n_tiles, const int* d_prefill_len, int window,
                        uocr_b200_workspace* ws, cudaStream_t st, const char* who) {
    if (!h_tiles || !d_prefill_len || !ws) return fail(UOCR_B200_ERR_INVALID, std::string(who) + ": null pointer");
    if (n_tiles <= 0 || window <= 0) return fail(UOCR_B200_ERR_INVALID, std::string(who) + ": tile count and window must be positive");
    if (n_tiles > ws->tiles_cap) return fail(UOCR_B200_ERR_WORKSPACE, std::string(who) + ": more tiles than the workspace holds");
    bool any_text = false;
    for (int i = 0; i < n_tiles; ++i) {
        const uocr_b200_prefill_tile& t = h_tiles[i];
        if (t.rows < 1 || t.rows > kTcTile || t.row0 < 0 || t.slot < 0 || t.pos0 < 0 || (t.kind != 0 && t.kind != 1))
            return fail(UOCR_B200_ERR_INVALID, std::string(who) + ": bad tile descriptor");
        any_text |= t.kind == 1;
    }
    static_assert(sizeof(uocr_b200_prefill_tile) == sizeof(PrefillTile), "tile descriptor layouts must match");
    ws->plan_tiles = 0;
    // pageable source: the copy has read the descriptors when the call returns
    CHECK_CUDA(cudaMemcpyAsync(ws->tiles, h_tiles, sizeof(PrefillTile) * (size_t)n_tiles, cudaMemcpyHostToDevice, st),
               "tile descriptors H2D");
    PrefillParams pp{};
    pp.tiles = ws->tiles;
    pp.n_tiles = n_tiles;
    pp.d_prefill_len = d_prefill_len;
    pp.window = window;
    rswa_prefill_order_kernel<<<1, 256, 0, st>>>(pp, ws->tile_work);
    if (int rc = after_launch("prefill tile order")) return rc;
    ws->plan_tiles = n_tiles;
    ws->plan_window = window;
    ws->plan_any_text = any_text;
    ++ws->plan_serial;
    return UOCR_B200_OK;
}

unsigned uocr_b200_workspace_prefill_plan_serial(const uocr_b200_workspace* ws) { return ws ? ws->plan_serial : 0u; }

int uocr_b200_rswa_prefill_plan_tc(const uocr_b200_prefill_tile* h_tiles, int n_tiles, const int* d_prefill_len, int window,
                                   uocr_b200_workspace* ws, uocr_b200_stream_t stream) {
    return prefill_plan(h_tiles, n_tiles, d_prefill_len, window, ws, reinterpret_cast<cudaStream_t>(stream), "prefill_plan_tc");
}

int uocr_b200_rswa_prefill_attention_tc(const uocr_b200_paged_kv* kv, const void* text_k_pool, const void* text_v_pool,
                                        int text_blocks, const float* q, const int* d_prefill_len,
                                        const uocr_b200_prefill_tile* h_tiles, int n_tiles, int window, int heads,
                                        float* out, uocr_b200_workspace* ws, uocr_b200_stream_t stream) {
    if (n_tiles <= 0) return UOCR_B200_OK;
    PagedView pv;
    if (int rc = paged_view(kv, &pv)) return rc;
    if (kv->dtype != UOCR_B200_BF16 || kv->head_dim != kTcTile)
        return fail(UOCR_B200_ERR_UNSUPPORTED, "prefill_attention_tc: needs bf16 KV and head_dim 128");
    if (!q || !out || !d_prefill_len || !ws) return fail(UOCR_B200_ERR_INVALID, "prefill_attention_tc: null pointer");
    if (!aligned16(q) || !aligned16(out)) return fail(UOCR_B200_ERR_INVALID, "prefill_attention_tc: q/out must be 16-byte aligned");
    if (heads <= 0 || heads % kv->kv_heads != 0) return fail(UOCR_B200_ERR_INVALID, "prefill_attention_tc: heads must be a multiple of kv_heads");
    if (window <= 0) return fail(UOCR_B200_ERR_INVALID, "prefill_attention_tc: window must be positive");
    const DeviceInfo* di = nullptr;
    if (int rc = device_info(&di)) return rc;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    if (h_tiles) {
        if (int rc = prefill_plan(h_tiles, n_tiles, d_prefill_len, window, ws, st, "prefill_attention_tc")) return rc;
    } else if (ws->plan_tiles != n_tiles || ws->plan_window != window) {
        return fail(UOCR_B200_ERR_INVALID, "prefill_attention_tc: no tiles given and the workspace holds no plan of this size and window");
    }
    if (ws->plan_any_text && (!text_k_pool || !text_v_pool || text_blocks <= 0))
        return fail(UOCR_B200_ERR_INVALID, "prefill_attention_tc: text tiles need the text pool");
    const bool any_text = ws->plan_any_text;
    CHECK_CUDA(cudaMemsetAsync(ws->item_counter, 0, sizeof(int), st), "prefill item counter");
    PrefillParams pp{};
    pp.q = q;
    pp.out = out;
    pp.out_bf16 = ws->out_bf16 ? 1 : 0;
    pp.k_pool = pv.k_pool;
    pp.v_pool = pv.v_pool;
    pp.k_text = static_cast<const uint8_t*>(text_k_pool);
    pp.v_text = static_cast<const uint8_t*>(text_v_pool);
    pp.table = pv.table;
    pp.d_prefill_len = d_prefill_len;
    pp.tiles = ws->tiles;
    pp.work = ws->tile_work;
    pp.counter = ws->item_counter;
    pp.n_tiles = n_tiles;
    pp.table_stride = pv.table_stride;
    pp.num_blocks = pv.num_blocks;
    pp.text_blocks = text_blocks;
    pp.heads = heads;
    pp.kv_heads = kv->kv_heads;
    pp.group = heads / kv->kv_heads;
    pp.window = window;
    pp.scale_log2e = (1.0f / std::sqrt(128.0f)) * 1.4426950408889634f;
    pp.status = ws->status;
    pp.wait_limit = ws->wait_limit;
    static bool configured[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (!configured[dev & 63]) {
        CHECK_CUDA(cudaFuncSetAttribute(rswa_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kTcSmemBytes),
                   "prefill smem attribute");
        configured[dev & 63] = true;
    }
    PrefillMaps maps;
    const long pool_rows = (long)kv->num_blocks * kv->kv_heads * kBlockTokens;
    const long text_rows = (long)text_blocks * kv->kv_heads * kBlockTokens;
    if (int rc = make_kv_map(&maps.k, pv.k_pool, pool_rows)) return rc;
    if (int rc = make_kv_map(&maps.v, pv.v_pool, pool_rows)) return rc;
    if (any_text) {
        if (int rc = make_kv_map(&maps.tk, text_k_pool, text_rows)) return rc;
        if (int rc = make_kv_map(&maps.tv, text_v_pool, text_rows)) return rc;
    } else {  // never read: no text tile in this launch
        maps.tk = maps.k;
        maps.tv = maps.v;
    }
    // the persistent grid: one CTA per SM draws (tile, head) items in the plan's order
    const long long n_items = (long long)n_tiles * heads;
    const int grid = (int)std::min<long long>(n_items, di->sms);
    rswa_prefill_tc_kernel<<<grid, kTcThreads, kTcSmemBytes, st>>>(pp, maps);
    return after_launch("tensor-core prefill attention");
}

// ---- fused decode step ---------------------------------------------------------------------------------
int uocr_b200_rswa_decode_step_paged(const uocr_b200_paged_kv* kv, const float* q, const float* k, const float* v,
                                     int* d_len, int* d_ring_pos, const int* d_prefill_len, const int* d_slots,
                                     int batch, int window, int heads, float* out, uocr_b200_workspace* ws,
                                     uocr_b200_stream_t stream) {
    if (batch <= 0) return UOCR_B200_OK;
    if (!k || !v || !d_len || !d_ring_pos || !d_prefill_len || !d_slots)
        return fail(UOCR_B200_ERR_INVALID, "decode_step_paged: null pointer");
    if (window <= 0) return fail(UOCR_B200_ERR_INVALID, "decode_step_paged: window must be positive");
    if (!aligned16(k) || !aligned16(v)) return fail(UOCR_B200_ERR_INVALID, "decode_step_paged: k/v must be 16-byte aligned");
    if (batch > kFusedMaxRows) {
        // too many rows to plan in shared memory: same result from the two separate launches
        if (int rc = uocr_b200_rswa_append_decode_batch_paged(kv, k, v, d_len, d_ring_pos, d_prefill_len, d_slots,
                                                              batch, window, ws, stream))
            return rc;
        return uocr_b200_rswa_attention_batch_paged(kv, q, d_len, d_prefill_len, d_slots, batch, heads, out, ws, stream);
    }
    AttnCall c;
    if (int rc = fill_paged(c, kv)) return rc;
    c.rows = batch; c.heads = heads; c.q = q; c.out = out;
    c.fused = true; c.k_new = k; c.v_new = v; c.d_len_rw = d_len; c.d_ring_rw = d_ring_pos;
    c.plan.mode = kPlanDecodeStep; c.plan.d_slots = d_slots; c.plan.d_len = d_len; c.plan.d_ring_pos = d_ring_pos;
    c.plan.d_prefill_len = d_prefill_len; c.plan.window = window;
    return run_attention(c, ws, reinterpret_cast<cudaStream_t>(stream));
}

int uocr_b200_rswa_decode_step_rope_paged(const uocr_b200_paged_kv* kv, const float* q, const float* k, const float* v,
                                          const int* d_positions, float theta, int* d_len, int* d_ring_pos,
                                          const int* d_prefill_len, const int* d_slots, int batch, int window, int heads,
                                          float* out, uocr_b200_workspace* ws, uocr_b200_stream_t stream) {
    if (batch <= 0) return UOCR_B200_OK;
    if (!k || !v || !d_positions || !d_len || !d_ring_pos || !d_prefill_len || !d_slots)
        return fail(UOCR_B200_ERR_INVALID, "decode_step_rope_paged: null pointer");
    if (window <= 0) return fail(UOCR_B200_ERR_INVALID, "decode_step_rope_paged: window must be positive");
    if (!(theta > 0.f)) return fail(UOCR_B200_ERR_INVALID, "decode_step_rope_paged: theta must be positive");
    if (!aligned16(k) || !aligned16(v)) return fail(UOCR_B200_ERR_INVALID, "decode_step_rope_paged: k/v must be 16-byte aligned");
    if (batch > kFusedMaxRows)
        return fail(UOCR_B200_ERR_UNSUPPORTED, "decode_step_rope_paged: at most 1024 rows per call");
    AttnCall c;
    if (int rc = fill_paged(c, kv)) return rc;
    c.rows = batch; c.heads = heads; c.q = q; c.out = out;
    c.fused = true; c.k_new = k; c.v_new = v; c.d_len_rw = d_len; c.d_ring_rw = d_ring_pos;
    c.rope_pos = d_positions; c.rope_theta = theta;
    c.plan.mode = kPlanDecodeStep; c.plan.d_slots = d_slots; c.plan.d_len = d_len; c.plan.d_ring_pos = d_ring_pos;
    c.plan.d_prefill_len = d_prefill_len; c.plan.window = window;
    return run_attention(c, ws, reinterpret_cast<cudaStream_t>(stream));
}

// ---- gather ---------------------------------------------------------------------------------------------
int uocr_b200_rswa_gather_paged(const uocr_b200_paged_kv* kv, const int* d_len, const int* d_prefill_len,
                                const int* d_slots, int n, int capacity_rows, void* out_k, void* out_v,
                                int out_dtype, uocr_b200_workspace* ws, uocr_b200_stream_t stream) {
    if (n <= 0 || capacity_rows <= 0) return UOCR_B200_OK;
    PagedView pv;
    if (int rc = paged_view(kv, &pv)) return rc;
    if (!d_len || !d_prefill_len || !d_slots || !out_k || !out_v) return fail(UOCR_B200_ERR_INVALID, "gather_paged: null pointer");
    if (!aligned16(out_k) || !aligned16(out_v)) return fail(UOCR_B200_ERR_INVALID, "gather_paged: outputs must be 16-byte aligned");
    if (out_dtype != UOCR_B200_F32 && out_dtype != kv->dtype) return fail(UOCR_B200_ERR_UNSUPPORTED, "gather_paged: out_dtype must be fp32 or the pool dtype");
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    int* status = ws ? ws->status : nullptr;
    dim3 grid(capacity_rows, n);
    uint8_t* ok = static_cast<uint8_t*>(out_k);
    uint8_t* ov = static_cast<uint8_t*>(out_v);
    if (kv->dtype == UOCR_B200_BF16) {
        if (out_dtype == UOCR_B200_F32)
            rswa_gather_paged_kernel<BF16, true><<<grid, 160, 0, st>>>(pv, d_len, d_prefill_len, d_slots, capacity_rows, ok, ov, status);
        else
            rswa_gather_paged_kernel<BF16, false><<<grid, 160, 0, st>>>(pv, d_len, d_prefill_len, d_slots, capacity_rows, ok, ov, status);
    } else {
        rswa_gather_paged_kernel<F32, false><<<grid, 160, 0, st>>>(pv, d_len, d_prefill_len, d_slots, capacity_rows, ok, ov, status);
    }
    return after_launch("gather (paged)");
}

int uocr_b200_rswa_gather_heads_paged(const uocr_b200_paged_kv* kv, const int* d_len, const int* d_prefill_len,
                                      const int* d_slots, int n, int capacity_rows, float* out_k, float* out_v,
                                      uocr_b200_workspace* ws, uocr_b200_stream_t stream) {
    if (n <= 0 || capacity_rows <= 0) return UOCR_B200_OK;
    PagedView pv;
    if (int rc = paged_view(kv, &pv)) return rc;
    if (!d_len || !d_prefill_len || !d_slots || !out_k || !out_v) return fail(UOCR_B200_ERR_INVALID, "gather_heads_paged: null pointer");
    if (!aligned16(out_k) || !aligned16(out_v)) return fail(UOCR_B200_ERR_INVALID, "gather_heads_paged: outputs must be 16-byte aligned");
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    int* status = ws ? ws->status : nullptr;
    dim3 grid(capacity_rows, n);
    uint8_t* ok = reinterpret_cast<uint8_t*>(out_k);
    uint8_t* ov = reinterpret_cast<uint8_t*>(out_v);
    if (kv->dtype == UOCR_B200_BF16)
        rswa_gather_paged_kernel<BF16, true, true><<<grid, 160, 0, st>>>(pv, d_len, d_prefill_len, d_slots, capacity_rows, ok, ov, status);
    else
        rswa_gather_paged_kernel<F32, false, true><<<grid, 160, 0, st>>>(pv, d_len, d_prefill_len, d_slots, capacity_rows, ok, ov, status);
    return after_launch("gather (paged, head-major)");
}

}  // extern "C"

// =================================================================================================
// Allocation-free batched decode attention.
//
// For hosts that cannot allocate device memory (the GPU is owned by their own arena, a plugin
// contract forbids it, or the implicit device synchronisation of cudaMalloc is unaffordable), the
// split-KV scratch lives in a file-scope device array instead of a uocr_b200_workspace.  The name
// `g_noalloc_scratch` is only a host-side handle in host code: the device address is looked up once
// per device with cudaGetSymbolAddress (with that device current) and that pointer is what the
// kernels receive.
// =================================================================================================
namespace {

constexpr int kNoAllocMaxRows = 1024;
constexpr int kNoAllocMaxHeadDim = 128;
constexpr int kNoAllocMaxSms = 160;
constexpr int kNoAllocMaxWarps = kNoAllocMaxSms * kMaxWarpsPerCta;
constexpr size_t na_up(size_t x) { return (x + 255) & ~size_t(255); }
constexpr size_t kNaStatus = 0;
constexpr size_t kNaRs = na_up(256);
constexpr size_t kNaInfo = kNaRs + na_up(sizeof(int) * (kNoAllocMaxRows + 1));
constexpr size_t kNaAcc = kNaInfo + na_up(sizeof(RowInfo) * kNoAllocMaxRows);
constexpr size_t kNaMl = kNaAcc + na_up(sizeof(float) * 2 * size_t(kNoAllocMaxWarps) * kNoAllocMaxHeadDim);
constexpr size_t kNaCnt = kNaMl + na_up(sizeof(float) * 4 * size_t(kNoAllocMaxWarps));
constexpr size_t kNaCntBytes = sizeof(int) * (size_t(kNoAllocMaxWarps) + 64);
constexpr size_t kNoAllocBytes = kNaCnt + na_up(kNaCntBytes);

static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocBytes];

unsigned char* g_noalloc_ptr[64] = {nullptr};  // device address of the array, per device ordinal

// Device address of the built-in scratch on the current device (looked up once per device).
int noalloc_base(unsigned char** base, int* dev_out) {
    int dev = 0;
    CHECK_CUDA(cudaGetDevice(&dev), "cudaGetDevice");
    if (dev < 0 || dev >= 64) return fail(UOCR_B200_ERR_NO_DEVICE, "device ordinal out of range");
    if (!g_noalloc_ptr[dev]) {
        void* p = nullptr;
        CHECK_CUDA(cudaGetSymbolAddress(&p, g_noalloc_scratch), "cudaGetSymbolAddress(scratch)");
        g_noalloc_ptr[dev] = static_cast<unsigned char*>(p);
    }
    *base = g_noalloc_ptr[dev];
    if (dev_out) *dev_out = dev;
    return UOCR_B200_OK;
}

}  // namespace

extern "C" int uocr_b200_rswa_attention_batch_paged_noalloc(
    const uocr_b200_paged_kv* kv, const float* q, const int* d_len, const int* d_prefill_len,
    const int* d_slots, int batch, int heads, float* out, uocr_b200_stream_t stream) {
    if (batch <= 0) return UOCR_B200_OK;
    // every argument is checked before the shared array is touched
    if (!d_len || !d_slots || !d_prefill_len) return fail(UOCR_B200_ERR_INVALID, "attention_batch_paged_noalloc: null index array");
    if (batch > kNoAllocMaxRows)
        return fail(UOCR_B200_ERR_WORKSPACE, "attention_batch_paged_noalloc: batch exceeds the built-in scratch (max 1024 rows)");
    AttnCall c;
    if (int rc = fill_paged(c, kv)) return rc;
    if (!kv->k_pool || !kv->v_pool || !q || !out) return fail(UOCR_B200_ERR_INVALID, "attention_batch_paged_noalloc: null pointer");
    if (kv->head_dim > kNoAllocMaxHeadDim)
        return fail(UOCR_B200_ERR_WORKSPACE, "attention_batch_paged_noalloc: head_dim exceeds the built-in scratch (max 128)");
    if (!head_dim_ok(kv->head_dim, kv->dtype)) return fail(UOCR_B200_ERR_UNSUPPORTED, "attention_batch_paged_noalloc: unsupported head_dim");
    if (heads <= 0 || kv->kv_heads <= 0 || heads % kv->kv_heads != 0)
        return fail(UOCR_B200_ERR_INVALID, "attention_batch_paged_noalloc: heads must be a positive multiple of kv_heads");
    const DeviceInfo* di = nullptr;
    if (int rc = device_info(&di)) return rc;
    if (di->sms > kNoAllocMaxSms)
        return fail(UOCR_B200_ERR_WORKSPACE, "attention_batch_paged_noalloc: device has more SMs than the built-in scratch covers (max 160)");

    // one-time set-up per device: resolve the device address of the static array
    unsigned char* base = nullptr;
    int dev = 0;
    if (int rc = noalloc_base(&base, &dev)) return rc;

    uocr_b200_workspace view;  // a view over the static array; owns nothing
    view.device = dev;
    view.max_rows = kNoAllocMaxRows;
    view.total_warps_max = kNoAllocMaxWarps;
    view.status = reinterpret_cast<int*>(base + kNaStatus);
    view.rs = reinterpret_cast<int*>(base + kNaRs);
    view.info = reinterpret_cast<RowInfo*>(base + kNaInfo);
    view.part_acc = reinterpret_cast<float*>(base + kNaAcc);
    view.part_ml = reinterpret_cast<float*>(base + kNaMl);
    view.counters = reinterpret_cast<int*>(base + kNaCnt);
    view.planned_ctas = view.counters + kNoAllocMaxWarps;
    view.pieces_max = kNoAllocMaxWarps;

    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    // One part of the scratch must start at zero: the arrival counters of the split items (the kernel
    // returns them to zero itself, but an earlier call that was cut short could have left some behind).
    // Everything else is rewritten before it is read.  The status word is NOT cleared here: faults
    // accumulate until uocr_b200_noalloc_status reads them.
    CHECK_CUDA(cudaMemsetAsync(view.counters, 0, kNaCntBytes, st), "scratch counter clear");

    c.rows = batch; c.heads = heads; c.q = q; c.out = out;
    c.plan.mode = kPlanBatch; c.plan.d_slots = d_slots; c.plan.d_len = d_len; c.plan.d_prefill_len = d_prefill_len;
    return run_attention(c, &view, st);
}

extern "C" int uocr_b200_noalloc_status(uocr_b200_stream_t stream, int* device_status) {
    if (!device_status) return fail(UOCR_B200_ERR_INVALID, "noalloc_status: null argument");
    unsigned char* base = nullptr;
    if (int rc = noalloc_base(&base, nullptr)) return rc;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    int v = 0;
    CHECK_CUDA(cudaMemcpyAsync(&v, base + kNaStatus, sizeof(int), cudaMemcpyDeviceToHost, st), "noalloc status D2H");
    CHECK_CUDA(cudaMemsetAsync(base + kNaStatus, 0, sizeof(int), st), "noalloc status clear");
    CHECK_CUDA(cudaStreamSynchronize(st), "noalloc status sync");
    *device_status = v;
    return UOCR_B200_OK;
}
