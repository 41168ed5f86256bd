// Host-side plumbing of libfrx: error text, device attributes, the HBM expert arena.
#include "frx_common.cuh"

#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <mutex>
#include <new>
#include <vector>

namespace frx {

namespace {
thread_local char g_err[512] = "";
}

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    std::vsnprintf(g_err, sizeof g_err, fmt, ap);
    va_end(ap);
    return code;
}

int cuda_fail(cudaError_t e, const char* what) {
    return fail(FRX_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

int sm_count() {
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    return n;
}

int max_smem_optin() {
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess) return 0;
    return n;
}

// ---- the limit of device-side waits
namespace {
std::atomic<unsigned long long> g_wait_limit_ns{kWaitLimitNs};
}
uint64_t wait_limit_ns() { return g_wait_limit_ns.load(std::memory_order_relaxed); }

// ---- per-kernel timing
bool g_profile_on = false;
namespace {
struct ProfRec {
    int cls;
    cudaEvent_t start, stop;
};
std::mutex g_prof_mu;
std::vector<ProfRec> g_prof;
std::vector<cudaEvent_t> g_prof_pool;
cudaEvent_t prof_event() {
    if (!g_prof_pool.empty()) {
        cudaEvent_t e = g_prof_pool.back();
        g_prof_pool.pop_back();
        return e;
    }
    cudaEvent_t e = nullptr;
    cudaEventCreate(&e);
    return e;
}
}  // namespace

void profile_mark(int cls, cudaStream_t stream, bool start) {
    std::lock_guard<std::mutex> lk(g_prof_mu);
    if (start) {
        ProfRec r{cls, prof_event(), prof_event()};
        cudaEventRecord(r.start, stream);
        g_prof.push_back(r);
    } else {
        for (size_t i = g_prof.size(); i-- > 0;)
            if (g_prof[i].cls == cls) {
                cudaEventRecord(g_prof[i].stop, stream);
                break;
            }
    }
}

}  // namespace frx

using namespace frx;

struct frx_arena {
    uint8_t* base = nullptr;
    size_t stride = 0, blob_bytes = 0;
    int n_layer = 0, n_expert = 0, n = 0, ff = 0;
    uint8_t* staging = nullptr;   // planar blobs on their way in
    int staging_blobs = 0;
};

extern "C" {

int frx_profile_begin(void) {
    std::lock_guard<std::mutex> lk(g_prof_mu);
    for (auto& r : g_prof) {
        g_prof_pool.push_back(r.start);
        g_prof_pool.push_back(r.stop);
    }
    g_prof.clear();
    g_profile_on = true;
    return FRX_OK;
}

int frx_profile_end(float* ms, int* launches, int n_classes) {
    std::lock_guard<std::mutex> lk(g_prof_mu);
    g_profile_on = false;
    if (!ms || !launches || n_classes < 1) return fail(FRX_ERR_ARG, "frx_profile_end: null output");
    for (int i = 0; i < n_classes; ++i) {
        ms[i] = 0.0f;
        launches[i] = 0;
    }
    int rc = FRX_OK;
    for (auto& r : g_prof) {
        float t = 0.0f;
        cudaError_t e = cudaEventSynchronize(r.stop);
        if (e == cudaSuccess) e = cudaEventElapsedTime(&t, r.start, r.stop);
        if (e != cudaSuccess) rc = cuda_fail(e, "frx_profile_end");
        else if (r.cls >= 0 && r.cls < n_classes) {
            ms[r.cls] += t;
            ++launches[r.cls];
        }
        g_prof_pool.push_back(r.start);
        g_prof_pool.push_back(r.stop);
    }
    g_prof.clear();
    return rc;
}

const char* frx_profile_class_name(int cls) {
    static const char* names[kNumKernelClasses] = {"route_topk", "quant_q8", "group", "gate_up", "down", "combine", "layout", "route_group_quant", "ffn"};
    return cls >= 0 && cls < kNumKernelClasses ? names[cls] : "";
}

int frx_version(void) { return 2; }

int frx_debug_set_wait_limit_ns(unsigned long long ns) {
    frx::g_wait_limit_ns.store(ns ? ns : frx::kWaitLimitNs, std::memory_order_relaxed);
    return FRX_OK;
}
const char* frx_last_error(void) { return g_err; }

size_t frx_q2_mat_bytes(int rows, int cols) { return size_t(rows) * size_t(cols / kQK) * kBlockBytes; }
size_t frx_q2_expert_bytes(int n, int ff) { return 2 * frx_q2_mat_bytes(ff, n) + frx_q2_mat_bytes(n, ff); }
size_t frx_q2_expert_stride(int n, int ff) { return align_up(frx_q2_expert_bytes(n, ff), 4096); }

int frx_arena_create(frx_arena** out, int n_layer, int n_expert, int n, int ff) {
    if (!out) return fail(FRX_ERR_ARG, "frx_arena_create: null out");
    if (n_layer < 1 || n_expert < 1) return fail(FRX_ERR_ARG, "frx_arena_create: n_layer %d, n_expert %d", n_layer, n_expert);
    if (n < kUnitK || ff < kUnitK || n % kUnitK || ff % kUnitK)
        return fail(FRX_ERR_SHAPE, "frx_arena_create: n %d and ff %d must be multiples of %d", n, ff, kUnitK);
    frx_arena* a = new (std::nothrow) frx_arena();
    if (!a) return fail(FRX_ERR_ARG, "frx_arena_create: out of host memory");
    a->n_layer = n_layer;
    a->n_expert = n_expert;
    a->n = n;
    a->ff = ff;
    a->blob_bytes = frx_q2_expert_bytes(n, ff);
    a->stride = frx_q2_expert_stride(n, ff);
    a->staging_blobs = 64;
    cudaError_t e = cudaMalloc(&a->base, size_t(n_layer) * n_expert * a->stride);
    if (e == cudaSuccess) e = cudaMalloc(&a->staging, size_t(a->staging_blobs) * a->stride);
    if (e != cudaSuccess) {
        cudaFree(a->base);
        delete a;
        return cuda_fail(e, "frx_arena_create: cudaMalloc");
    }
    *out = a;
    return FRX_OK;
}

int frx_arena_destroy(frx_arena* a) {
    if (!a) return FRX_OK;
    cudaFree(a->base);
    cudaFree(a->staging);
    delete a;
    return FRX_OK;
}

void* frx_arena_base(const frx_arena* a) { return a ? a->base : nullptr; }
void* frx_arena_blob(const frx_arena* a, int layer, int expert) {
    if (!a || layer < 0 || layer >= a->n_layer || expert < 0 || expert >= a->n_expert) return nullptr;
    return a->base + (size_t(layer) * a->n_expert + expert) * a->stride;
}
size_t frx_arena_stride(const frx_arena* a) { return a ? a->stride : 0; }
size_t frx_arena_total_bytes(const frx_arena* a) { return a ? size_t(a->n_layer) * a->n_expert * a->stride : 0; }

int frx_arena_load_planar(frx_arena* a, int layer, int expert0, int count, const void* src_planar, size_t src_stride,
                          frx_stream_t stream) {
    if (!a || !src_planar) return fail(FRX_ERR_ARG, "frx_arena_load_planar: null argument");
    if (layer < 0 || layer >= a->n_layer || expert0 < 0 || count < 0 || expert0 + count > a->n_expert)
        return fail(FRX_ERR_ARG, "frx_arena_load_planar: layer %d, experts [%d, %d) outside the arena", layer, expert0, expert0 + count);
    if (src_stride < a->blob_bytes) return fail(FRX_ERR_ARG, "frx_arena_load_planar: src_stride %zu < blob %zu", src_stride, a->blob_bytes);
    const auto* src = static_cast<const uint8_t*>(src_planar);
    for (int done = 0; done < count;) {
        const int nb = count - done < a->staging_blobs ? count - done : a->staging_blobs;
        FRX_CUDA(cudaMemcpy2DAsync(a->staging, a->stride, src + size_t(done) * src_stride, src_stride, a->blob_bytes, nb,
                                   cudaMemcpyDefault, stream));
        const int rc = frx_q2_tile_experts(a->staging, a->stride, frx_arena_blob(a, layer, expert0 + done), a->stride, nb, a->n,
                                           a->ff, stream);
        if (rc) return rc;
        done += nb;
    }
    return FRX_OK;
}

}  // extern "C"
