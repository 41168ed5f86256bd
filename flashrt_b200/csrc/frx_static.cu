// frx_moe_decode_static: the decode-sized MoE layer for callers that may not allocate device memory.
//
// Some hosts of this library cannot hand it a workspace: an engine that gave every free byte of
// device memory to its caches when it started (the reference sizes its expert cache from whatever
// is free at start-up), a real-time loop whose rules forbid cudaMalloc after initialisation, or a
// plugin host that owns the allocator. For them the workspace of frx_moe_decode lives here, in a
// fixed array inside the library's device image. Every GPU that loads libfrx holds these
// kStaticScratchBytes until the process exits, whether or not this entry point is ever called.
#include "frx_common.cuh"

#include <mutex>

namespace {

constexpr size_t kStaticScratchBytes = size_t(4) << 20;   // 4 MiB

// The workspace. In host code this name is only a handle for the runtime (it is not a device
// address and must never be passed to a kernel); the device address comes from
// cudaGetSymbolAddress, asked once per device with that device current.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_mu;
void* g_scratch_addr[kMaxDevices] = {};

// Device address of g_static_scratch on the current device.
int scratch_address(void** out) {
    int dev = 0;
    FRX_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return frx::fail(FRX_ERR_ARG, "frx_moe_decode_static: device ordinal %d not supported", dev);
    std::lock_guard<std::mutex> lk(g_mu);
    if (!g_scratch_addr[dev]) {
        void* p = nullptr;
        FRX_CUDA(cudaGetSymbolAddress(&p, g_static_scratch));
        g_scratch_addr[dev] = p;
    }
    *out = g_scratch_addr[dev];
    return FRX_OK;
}

}  // namespace

extern "C" int frx_moe_decode_static(const void* experts, size_t stride, int E, const void* shared, int n, int ff, const float* x,
                                     const int32_t* ids, const float* wts, const float* gate_logit, int T, int K, float* out,
                                     frx_stream_t stream) {
    if (T < 0) return frx::fail(FRX_ERR_ARG, "frx_moe_decode_static: T %d", T);
    if (T == 0) return FRX_OK;
    const size_t need = frx_moe_decode_workspace_bytes(T, K, n, ff);
    if (need == 0) return frx::fail(FRX_ERR_SHAPE, "frx_moe_decode_static: unsupported shape T %d, K %d, n %d, ff %d", T, K, n, ff);
    if (need > kStaticScratchBytes)
        return frx::fail(FRX_ERR_WORKSPACE,
                         "frx_moe_decode_static: T %d x K %d at n %d, ff %d needs %zu bytes of scratch, the built-in scratch holds %zu; "
                         "use frx_moe_decode with a workspace of your own",
                         T, K, n, ff, need, kStaticScratchBytes);
    void* scratch = nullptr;
    if (int rc = scratch_address(&scratch)) return rc;
    // The array keeps whatever the previous call left. The layer's kernels rewrite every buffer
    // they read, and the status words at its start are (re)initialised by the grouping kernel
    // when they do not carry its cookie, which a zero-filled, freshly loaded array does not.
    return frx_moe_decode(experts, stride, E, shared, n, ff, x, ids, wts, gate_logit, T, K, out, nullptr, scratch, kStaticScratchBytes,
                          stream);
}

// The status of the built-in scratch: FRX_OK, or FRX_ERR_DEVICE if a kernel of an earlier
// frx_moe_decode_static call on this device reported an error (a bad expert id, a wait that ran
// out); reading the error clears it. Synchronises the stream; allocates nothing.
extern "C" int frx_moe_decode_static_status(frx_stream_t stream) {
    void* scratch = nullptr;
    if (int rc = scratch_address(&scratch)) return rc;
    return frx_workspace_status(scratch, stream);
}
