// The join between the layers of the chained expert-stack benchmark (48 MoE layers, a window of
// three tokens per step): x_next = (x + y) / sqrt(mean((x + y)^2) + 1e-6), an RMS norm with unit
// weight. The reference joins its MoE layers through its attention blocks, which are outside this
// library; this stand-in keeps the activations of a deep stack at unit scale so that every layer
// sees realistic inputs. The order of every floating-point operation is fixed and stated, so a CPU
// restatement gives the same bits: r = x + y in float; lane l of one warp adds r[l]^2, r[l + 32]^2,
// ... in double in that order; the 32 lane sums are combined by a butterfly (offsets 16, 8, 4, 2,
// 1); inv = float(1 / sqrt(sum / n + 1e-6)) in double; x_next = r * inv in float.
#include "frx_common.cuh"

namespace frx {
namespace {

__global__ void __launch_bounds__(32) k_chain_rmsnorm(const float* __restrict__ x, const float* __restrict__ y, float* __restrict__ out, int n) {
    pdl_wait();
    pdl_trigger();
    const int t = blockIdx.x, lane = threadIdx.x;
    const float* xr = x + size_t(t) * n;
    const float* yr = y + size_t(t) * n;
    double ss = 0.0;
    for (int i = lane; i < n; i += 32) {
        const float r = __fadd_rn(xr[i], yr[i]);
        ss = __dadd_rn(ss, __dmul_rn(double(r), double(r)));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss = __dadd_rn(ss, __shfl_xor_sync(0xffffffffu, ss, o));
    const float inv = float(__ddiv_rn(1.0, __dsqrt_rn(__dadd_rn(__ddiv_rn(ss, double(n)), 1e-6))));
    for (int i = lane; i < n; i += 32) out[size_t(t) * n + i] = __fmul_rn(__fadd_rn(xr[i], yr[i]), inv);
}

}  // namespace
}  // namespace frx

using namespace frx;

extern "C" int frx_chain_rmsnorm_unit(const float* x, const float* y, float* x_next, int T, int n, frx_stream_t stream) {
    if (T < 0 || n < 1) return fail(FRX_ERR_ARG, "frx_chain_rmsnorm_unit: T %d, n %d", T, n);
    if (T == 0) return FRX_OK;
    if (!x || !y || !x_next) return fail(FRX_ERR_ARG, "frx_chain_rmsnorm_unit: null pointer");
    FRX_LAUNCH(kKCombine, stream, launch_pdl(k_chain_rmsnorm, dim3(unsigned(T)), dim3(32), 0, stream, x, y, x_next, n));
    FRX_CUDA(cudaGetLastError());
    return FRX_OK;
}
