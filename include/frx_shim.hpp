// The reference's own C++ signatures for the Q2_0 MoE expert path, implemented over libfrx's C ABI.
// A reference call site (arch/qwen4exp/moe_stream.cu:164-166, moe_fast.cu:1044-1072, mtp.cu:636-666)
// that includes this header instead of kernels/cuda/moe_q2.h, arch/qwen4exp/moe_fast.hpp and the
// routing declaration of arch/qwen4exp/blocks.hpp compiles unchanged and links against libfrx.so.
// Errors become std::runtime_error, as in the reference (kernels/cuda/moe_q2.cu:516-519).
//
// Differences a caller must know:
//   - expert blobs are in libfrx's tiled layout (frx_q2_tile_experts / frx_arena_load_planar), not
//     the planar layout of quant/q2_0/q2_0.hpp;
//   - activations are always quantized per 32 values with round-half-away (the CPU path's rule):
//     moe_q2::run rejects block64 = true, and moe_hits does not reproduce the per-64
//     round-half-even of the reference's decode kernel;
//   - moe_q2::run writes float outputs only (yd_bf16 = true is rejected).
#pragma once

#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>
#include <stdexcept>
#include <string>

#include "frx.h"

namespace flashrt {

namespace frx_detail {
inline void check(int rc, const char* who) {
    if (rc != FRX_OK) throw std::runtime_error(std::string(who) + ": " + frx_last_error());
}
constexpr int kMaxModelDim = 8192;   // moe_hits_scratch_bytes is not told d_model: size for the largest
}  // namespace frx_detail

namespace moe_q2 {   // kernels/cuda/moe_q2.h:21-30

inline size_t workspace_bytes(int T, int K, int n, int ff, int E) { return frx_moe_prefill_workspace_bytes(T, K, n, ff, E); }

inline void run(const uint8_t* experts, size_t stride, int E, int n, int ff, const float* x, const int32_t* ids, int T, int K,
                void* yd, void* ws, size_t ws_bytes, cudaStream_t stream, bool block64 = false, bool yd_bf16 = false) {
    if (block64 || yd_bf16) throw std::runtime_error("moe_q2::run: block64 and yd_bf16 are not supported by libfrx");
    frx_detail::check(frx_moe_prefill(experts, stride, E, n, ff, x, ids, T, K, static_cast<float*>(yd), ws, ws_bytes, stream),
                      "moe_q2::run");
}

}  // namespace moe_q2

namespace qwen4exp {

// arch/qwen4exp/blocks.hpp:134-135
inline void moe_route_topk(cudaStream_t stream, const float* logits, int T, int E, int k, int32_t* ids, float* wts,
                           uint32_t* counts, uint32_t* tail_counts = nullptr, int tail_from = 1 << 30) {
    frx_detail::check(frx_route_topk(stream, logits, T, E, k, ids, wts, counts, tail_counts, tail_from), "moe_route_topk");
}

// arch/qwen4exp/moe_fast.hpp:140-142
inline size_t moe_hits_scratch_bytes(int K, int ff, int T = 1) {
    return frx_moe_hits_scratch_bytes(K, frx_detail::kMaxModelDim, ff, T);
}
inline void moe_hits(const uint8_t* const* hit_ptr, const int32_t* hit_n, int K, const float* x, int n, int ff, void* scratch,
                     float* yh, cudaStream_t stream, int T = 1) {
    frx_detail::check(frx_moe_hits(hit_ptr, hit_n, K, x, n, ff, scratch, moe_hits_scratch_bytes(K, ff, T), yh, stream, T), "moe_hits");
}

}  // namespace qwen4exp

}  // namespace flashrt
