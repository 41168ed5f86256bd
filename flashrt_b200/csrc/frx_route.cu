// Router entry point; the device code is in frx_route.cuh.
#include "frx_route.cuh"

namespace frx {
namespace {

template <int V>
__global__ void __launch_bounds__(256) k_route_topk(const float* __restrict__ logits, int T, int E, int K, int32_t* __restrict__ ids,
                                                    float* __restrict__ wts, uint32_t* counts, uint32_t* tail, int tail_from) {
    pdl_wait();
    pdl_trigger();
    const int t = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (t >= T) return;
    route_warp<V>(logits + size_t(t) * E, E, K, lane, ids + size_t(t) * K, wts + size_t(t) * K, counts, (tail && t >= tail_from) ? tail : nullptr);
}

}  // namespace
}  // namespace frx

using namespace frx;

extern "C" int frx_route_topk(frx_stream_t stream, const float* logits, int T, int E, int k, int32_t* ids, float* wts,
                              uint32_t* counts, uint32_t* tail_counts, int tail_from) {
    if (!logits || !ids || !wts) return fail(FRX_ERR_ARG, "frx_route_topk: null pointer");
    if (T < 0) return fail(FRX_ERR_ARG, "frx_route_topk: T %d", T);
    if (E < 1 || E > 1024 || k < 1 || k > 32 || k > E) return fail(FRX_ERR_SHAPE, "frx_route_topk: unsupported shape E %d, k %d", E, k);
    if (T == 0) return FRX_OK;
    const unsigned grid = unsigned((T + 7) / 8);
    if (E <= 128)
        FRX_LAUNCH(kKRoute, stream, launch_pdl(k_route_topk<4>, dim3(grid), dim3(256), 0, stream, logits, T, E, k, ids, wts, counts, tail_counts, tail_from));
    else if (E <= 512)
        FRX_LAUNCH(kKRoute, stream, launch_pdl(k_route_topk<16>, dim3(grid), dim3(256), 0, stream, logits, T, E, k, ids, wts, counts, tail_counts, tail_from));
    else
        FRX_LAUNCH(kKRoute, stream, launch_pdl(k_route_topk<32>, dim3(grid), dim3(256), 0, stream, logits, T, E, k, ids, wts, counts, tail_counts, tail_from));
    FRX_CUDA(cudaGetLastError());
    return FRX_OK;
}
