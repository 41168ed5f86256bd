// Router projection in front of the router: logits[t][e] = sum_k W[e][k] * x[t][k], with W in bf16
// and x, the products and the sums in fp32, and in the same launch the shared expert's gate logit
// (one more bf16 row). The reference computes both with one launch of k_bf16_multi
// (arch/qwen4exp/blocks.cu:83-120, called at moe_fast.cu:1039-1042 and moe_stream.cu:145-149): exact
// bf16 x fp32 products, fp32 accumulation, no activation on these two outputs. The order of the
// additions differs from the reference's (and from one GPU generation's launch shape to another in
// the reference itself), so parity is to a tolerance, against a float64 sum.
//
// One block = 8 output rows x 64 tokens. Each of its 8 warps takes an eighth of K and walks it in
// pieces of 32: the piece of x (64 tokens x 32 values) and of W (8 rows x 32 bf16) go through the
// warp's own shared memory (cp.async, the next piece in flight while this one is used), a lane accumulates 4 rows x 4 tokens from
// 16-byte loads, and at the end the eight partial tiles are added in warp order (fixed, so results
// are reproducible).
#include "frx_common.cuh"

#include <mutex>

namespace frx {
namespace {

constexpr int kRtRows = 8, kRtTok = 64, kRtWarps = 8, kRtPiece = 32, kRtPad = 36;   // 36: rows stay 16-byte aligned, no bank conflicts
constexpr int kRtPieceBytes = kRtTok * kRtPad * 4 + kRtRows * kRtPiece * 2;          // x piece (fp32, padded rows) + W piece (bf16)
constexpr int kRtSmemWarp = 2 * kRtPieceBytes;                                       // two pieces: one in flight, one in use
constexpr int kRtSmem = kRtWarps * kRtSmemWarp;

__device__ __forceinline__ float bf16_lo(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t u) { return __uint_as_float(u & 0xffff0000u); }
// 16 bytes global -> shared without passing through registers; src_bytes = 0 writes zeros
__device__ __forceinline__ void cp_async16(void* dst, const void* src, uint32_t src_bytes) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// rows: E router rows followed by the gate row when w_gate is given (row E). W rows are n bf16 each.
__global__ void __launch_bounds__(kRtWarps * 32) k_router_logits(const uint16_t* __restrict__ w_router, const uint16_t* __restrict__ w_gate,
                                                                  const float* __restrict__ x, int T, int E, int n,
                                                                  float* __restrict__ logits, float* __restrict__ gate_logit) {
    extern __shared__ __align__(16) uint8_t smem[];
    pdl_wait();
    pdl_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint8_t* mine = smem + warp * kRtSmemWarp;
    const int rows_total = E + (w_gate ? 1 : 0);
    const int r0 = blockIdx.x * kRtRows, t0 = blockIdx.y * kRtTok;
    const int ry = lane >> 4, tx = lane & 15;   // this lane's tile: rows 4 ry .. + 3, tokens tx, tx + 16, tx + 32, tx + 48 (no bank conflicts)
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;
    const int kslice = n / kRtWarps, pieces = kslice / kRtPiece, kbase = warp * kslice;
    // the copy of one piece into buffer `buf`: 64 tokens x 8 float4 of x, 8 rows x 32 bf16 of W
    auto fetch = [&](int piece, int buf) {
        const int k0 = kbase + piece * kRtPiece;
        float* xs = reinterpret_cast<float*>(mine + buf * kRtPieceBytes);
        uint16_t* wsb = reinterpret_cast<uint16_t*>(mine + buf * kRtPieceBytes + kRtTok * kRtPad * 4);
#pragma unroll
        for (int it = 0; it < 16; ++it) {
            const int idx = it * 32 + lane, tok = idx >> 3, k4 = idx & 7;
            const bool in = t0 + tok < T;
            cp_async16(xs + tok * kRtPad + k4 * 4, x + size_t(in ? t0 + tok : 0) * n + k0 + k4 * 4, in ? 16u : 0u);
        }
        const int row = lane >> 2, k8 = (lane & 3) * 8, r = r0 + row;
        const uint16_t* src = r < E ? w_router + size_t(r) * n + k0 + k8 : w_gate ? w_gate + k0 + k8 : w_router + k0 + k8;
        cp_async16(wsb + row * kRtPiece + k8, src, r < rows_total ? 16u : 0u);
        cp_async_commit();
    };
    fetch(0, 0);
    for (int piece = 0; piece < pieces; ++piece) {
        const int buf = piece & 1;
        if (piece + 1 < pieces) {
            fetch(piece + 1, buf ^ 1);
            cp_async_wait<1>();   // everything but the copy just started has landed
        } else {
            cp_async_wait<0>();
        }
        __syncwarp();
        const float* xs = reinterpret_cast<const float*>(mine + buf * kRtPieceBytes);
        const uint16_t* wsb = reinterpret_cast<const uint16_t*>(mine + buf * kRtPieceBytes + kRtTok * kRtPad * 4);
#pragma unroll
        for (int k4 = 0; k4 < kRtPiece / 4; ++k4) {
            float4 wv[4], xv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint2 u = *reinterpret_cast<const uint2*>(wsb + (4 * ry + i) * kRtPiece + k4 * 4);
                wv[i] = make_float4(bf16_lo(u.x), bf16_hi(u.x), bf16_lo(u.y), bf16_hi(u.y));
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) xv[j] = *reinterpret_cast<const float4*>(xs + (tx + 16 * j) * kRtPad + k4 * 4);
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    acc[i][j] = fmaf(wv[i].x, xv[j].x, acc[i][j]);
                    acc[i][j] = fmaf(wv[i].y, xv[j].y, acc[i][j]);
                    acc[i][j] = fmaf(wv[i].z, xv[j].z, acc[i][j]);
                    acc[i][j] = fmaf(wv[i].w, xv[j].w, acc[i][j]);
                }
        }
        __syncwarp();   // the buffer is refilled by the fetch of the next iteration
    }
    // the eight K-slices: partial tiles to shared memory (the pieces are no longer needed), then one
    // thread per (row, token) adds them in warp order
    __syncthreads();
    float* red = reinterpret_cast<float*>(smem);   // [warp][8 rows][64 tokens]
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) red[(warp * kRtRows + 4 * ry + i) * kRtTok + tx + 16 * j] = acc[i][j];
    __syncthreads();
    for (int o = threadIdx.x; o < kRtRows * kRtTok; o += kRtWarps * 32) {
        const int row = o / kRtTok, tok = o % kRtTok, r = r0 + row, t = t0 + tok;
        float sum = red[o];
#pragma unroll
        for (int w = 1; w < kRtWarps; ++w) sum += red[w * kRtRows * kRtTok + o];
        if (t < T) {
            if (r < E) logits[size_t(t) * E + r] = sum;
            else if (r < rows_total && gate_logit) gate_logit[t] = sum;
        }
    }
}
static_assert(kRtWarps * kRtRows * kRtTok * 4 <= kRtSmem, "the reduction buffer reuses the pieces' shared memory");

}  // namespace
}  // namespace frx

using namespace frx;

extern "C" int frx_router_logits(frx_stream_t stream, const void* w_router, const void* w_gate, const float* x, int T, int E, int n,
                                 float* logits, float* gate_logit) {
    if (!w_router || !x || !logits) return fail(FRX_ERR_ARG, "frx_router_logits: null pointer");
    if (w_gate && !gate_logit) return fail(FRX_ERR_ARG, "frx_router_logits: gate weights without a gate output");
    if (T < 0 || E < 1 || n < 256 || n % 256) return fail(FRX_ERR_SHAPE, "frx_router_logits: T %d, E %d, n %d (n a multiple of 256)", T, E, n);
    if ((uintptr_t(w_router) | uintptr_t(w_gate) | uintptr_t(x)) % 16) return fail(FRX_ERR_ARG, "frx_router_logits: pointers must be 16-byte aligned");
    if (T == 0) return FRX_OK;
    static std::once_flag once[64];
    int dev = 0;
    FRX_CUDA(cudaGetDevice(&dev));
    cudaError_t attr = cudaSuccess;
    if (dev >= 0 && dev < 64)
        std::call_once(once[dev], [&] { attr = cudaFuncSetAttribute(k_router_logits, cudaFuncAttributeMaxDynamicSharedMemorySize, kRtSmem); });
    if (attr != cudaSuccess) return cuda_fail(attr, "frx_router_logits: cudaFuncSetAttribute");
    const int rows_total = E + (w_gate ? 1 : 0);
    const dim3 grid(unsigned((rows_total + kRtRows - 1) / kRtRows), unsigned((T + kRtTok - 1) / kRtTok));
    FRX_LAUNCH(kKRoute, stream, launch_pdl(k_router_logits, grid, dim3(kRtWarps * 32), size_t(kRtSmem), stream, static_cast<const uint16_t*>(w_router),
                                            static_cast<const uint16_t*>(w_gate), x, T, E, n, logits, gate_logit));
    FRX_CUDA(cudaGetLastError());
    return FRX_OK;
}
