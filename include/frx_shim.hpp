// The reference's own C++ signatures for the Q2_0 MoE expert path, implemented over libfrx's C ABI.
// A reference call site (arch/qwen4exp/moe_stream.cu:164-166, moe_fast.cu:1044-1072, mtp.cu:636-666)
// that includes this header instead of kernels/cuda/moe_q2.h, arch/qwen4exp/moe_fast.hpp and the
// routing declaration of arch/qwen4exp/blocks.hpp compiles unchanged and links against libfrx.so.
// Errors become std::runtime_error, as in the reference (kernels/cuda/moe_q2.cu:516-519).
//
// Differences a caller must know:
//   - expert blobs are in libfrx's tiled layout (frx_q2_tile_experts / frx_arena_load_planar), not
//     the planar layout of quant/q2_0/q2_0.hpp;
//   - activations are quantized per 32 values with round-half-away (the CPU path's rule) unless
//     moe_q2::run is given block64 = true (one scale per 64 values); moe_hits does not reproduce
//     the per-64 round-half-even of the reference's decode kernel;
//   - gemv:: and gemm:: take ggml type 42 (Q2_0) only; gemm::moe_prepare does not wait for the
//     stream, so MoePlan::ncols_max / ncols_opt are not filled in (nothing outside the reference's
//     own moe_run reads them).
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
    frx_detail::check(frx_moe_prefill_ex(experts, stride, E, n, ff, x, ids, T, K, yd, ws, ws_bytes, stream, block64 ? 1 : 0, yd_bf16 ? 1 : 0),
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

// arch/qwen4exp/mtp.hpp:40 (host buffers in the reference; device buffers here, on `stream`)
inline void convert_q8_0_to_q2_0_device(const uint8_t* src, uint8_t* dst, size_t nblocks64, cudaStream_t stream) {
    frx_detail::check(frx_convert_q8_0_to_q2_0(src, dst, nblocks64, stream), "convert_q8_0_to_q2_0");
}

}  // namespace qwen4exp

namespace gemv {   // kernels/cuda/ggml_gemv.h:19-65, ggml type 42 only

constexpr int kMaxTokens = 8;
constexpr size_t kWeightTailPad = 64 * 1024;   // libfrx reads nothing past the weights; kept for callers that size buffers with it

inline bool supported(uint32_t ggml_type) { return ggml_type == 42; }
inline bool is_float(uint32_t) { return false; }
inline int64_t row_bytes(uint32_t ggml_type, int64_t ncols) { return frx_gemv_row_bytes(ggml_type, ncols); }
inline size_t q8_1_bytes(int64_t ncols, int n_tok) { return frx_gemv_q8_1_bytes(ncols, n_tok); }
inline void quantize_q8_1(const float* x, int64_t ncols, int n_tok, void* xq, cudaStream_t stream) {
    frx_detail::check(frx_gemv_quantize_q8_1(x, ncols, n_tok, xq, stream), "gemv::quantize_q8_1");
}
inline void swiglu_q8_1(const float* g, const float* u, int64_t ncols, int n_tok, void* xq, cudaStream_t stream) {
    frx_detail::check(frx_gemv_swiglu_q8_1(g, u, ncols, n_tok, xq, stream), "gemv::swiglu_q8_1");
}
inline void matvec_q(uint32_t ggml_type, const void* W, const void* xq, float* y, int64_t ncols, int64_t nrows, int n_tok,
                     cudaStream_t stream) {
    frx_detail::check(frx_gemv_matvec_q(ggml_type, W, xq, y, ncols, nrows, n_tok, stream), "gemv::matvec_q");
}
inline void matvec(uint32_t ggml_type, const void* W, const float* x, float* y, int64_t ncols, int64_t nrows, int n_tok, void* scratch,
                   cudaStream_t stream) {
    frx_detail::check(frx_gemv_matvec(ggml_type, W, x, y, ncols, nrows, n_tok, scratch, stream), "gemv::matvec");
}
inline void moe_q2_0(const void* w, const void* gate, const void* xq, const int32_t* ids, float* dst, int n_ids, int64_t ncols,
                     int64_t nrows, int64_t slot_stride_bytes, bool per_channel_act, cudaStream_t stream) {
    frx_detail::check(frx_gemv_moe_q2_0(w, gate, xq, ids, dst, n_ids, ncols, nrows, slot_stride_bytes, per_channel_act ? 1 : 0, stream),
                      "gemv::moe_q2_0");
}
inline void moe_q(uint32_t ggml_type, const void* w, const void* gate, const void* xq, const int32_t* ids, float* dst, int n_tok, int k,
                  int64_t ncols, int64_t nrows, int64_t expert_stride_bytes, bool act_per_expert, cudaStream_t stream) {
    frx_detail::check(frx_gemv_moe_q(ggml_type, w, gate, xq, ids, dst, n_tok, k, ncols, nrows, expert_stride_bytes, act_per_expert ? 1 : 0, stream),
                      "gemv::moe_q");
}

}  // namespace gemv

namespace gemm {   // kernels/cuda/ggml_gemm.h:27-68, the grouped expert products, ggml type 42 only

inline bool supported(uint32_t ggml_type) { return ggml_type == 42; }
inline size_t workspace_bytes(int64_t ncols, int64_t T, bool /*bf16*/ = true) { return frx_gemm_workspace_bytes(ncols, T); }

struct MoePlan {   // the reference's fields, so that code which copies or inspects a plan still compiles
    uint32_t type = 0;
    int n_experts = 0, K = 0;
    int64_t T = 0, ncols = 0, rows = 0, ne11 = 0, ncols_max = 0, ncols_opt = 0;
    const int* act = nullptr;
    const int32_t *ids_dst = nullptr, *bounds = nullptr;
    float* fixup = nullptr;
    frx_gemm_moe_plan frx{};   // what libfrx's moe_run reads
};
inline MoePlan moe_prepare(uint32_t ggml_type, int n_experts, const float* x, bool x_per_slot, const int32_t* ids, int64_t T, int K,
                           int64_t ncols, void* ws, size_t ws_bytes, cudaStream_t stream) {
    MoePlan p;
    frx_detail::check(frx_gemm_moe_prepare(&p.frx, ggml_type, n_experts, x, x_per_slot ? 1 : 0, ids, T, K, ncols, ws, ws_bytes, stream),
                      "gemm::moe_prepare");
    p.type = ggml_type;
    p.n_experts = n_experts;
    p.K = K;
    p.T = T;
    p.ncols = ncols;
    p.rows = T * K;
    p.ne11 = x_per_slot ? K : 1;
    return p;
}
inline void moe_run(const MoePlan& plan, const void* W, int64_t expert_stride_bytes, float* y, int64_t nrows, cudaStream_t stream) {
    frx_detail::check(frx_gemm_moe_run(&plan.frx, W, expert_stride_bytes, y, nrows, stream), "gemm::moe_run");
}
inline void moe(uint32_t ggml_type, const void* W, int64_t expert_stride_bytes, int n_experts, const float* x, bool x_per_slot,
                const int32_t* ids, int64_t T, int K, float* y, int64_t ncols, int64_t nrows, void* ws, size_t ws_bytes,
                cudaStream_t stream) {
    frx_detail::check(frx_gemm_moe(ggml_type, W, expert_stride_bytes, n_experts, x, x_per_slot ? 1 : 0, ids, T, K, y, ncols, nrows, ws, ws_bytes,
                                   stream),
                      "gemm::moe");
}

}  // namespace gemm

}  // namespace flashrt
