// C entry points over the reference's own CPU sources, which are compiled where they lie in the
// reference tree (see the Makefile beside this file) and are never copied. TEST INFRASTRUCTURE
// ONLY: it validates the scalar oracle in q2_oracle.c and is the timed CPU baseline. Nothing in
// the product may link or load it.
//
// The code below only builds the call arguments. The Miss list follows what the reference's
// moe_block does before it calls q2_0::moe_cpu (arch/qwen4exp/moe_ref.cu:171-183): experts in
// ascending id, each expert's tokens in token order, at most four tokens per entry.
#include "core/cpu_pool.hpp"
#include "core/fp16.hpp"
#include "core/platform.hpp"
#include "quant/q2_0/moe_cpu.hpp"
#include "quant/q2_0/q2_0.hpp"

#include <chrono>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <utility>
#include <vector>

using namespace flashrt;
using namespace flashrt::q2_0;

namespace {

struct Acts {
    std::vector<uint8_t> mem;
    std::vector<Q8Act> a;
    Acts(const float* x, int T, int n) : mem(size_t(T) * q8_bytes(n) + 64), a(T) {
        auto p = (reinterpret_cast<uintptr_t>(mem.data()) + 63) & ~uintptr_t(63);
        for (int t = 0; t < T; ++t) {
            a[t] = q8_view(reinterpret_cast<void*>(p + size_t(t) * q8_bytes(n)), n);
            quantize_q8(x + size_t(t) * n, a[t]);
        }
    }
};

std::unique_ptr<CpuPool> g_pool;
int g_pool_n = 0;

CpuPool& pool(int workers) {
    if (!g_pool || g_pool_n != workers) {
        g_pool.reset();
        g_pool = std::make_unique<CpuPool>(workers, physical_cpus());
        g_pool_n = workers;
    }
    return *g_pool;
}

std::vector<Miss> build_entries(const uint8_t* experts, size_t stride, int E, const int32_t* ids, const float* wts, int T,
                                int K) {
    std::vector<std::vector<std::pair<int, float>>> routed(E);
    for (int t = 0; t < T; ++t)
        for (int k = 0; k < K; ++k) routed[ids[size_t(t) * K + k]].push_back({t, wts[size_t(t) * K + k]});
    std::vector<Miss> miss;
    for (int e = 0; e < E; ++e) {
        const auto& r = routed[e];
        for (size_t i = 0; i < r.size(); i += 4) {
            Miss m{experts + size_t(e) * stride, 0, {}, {}};
            for (size_t j = i; j < std::min(r.size(), i + 4); ++j) {
                m.tok[m.n_tok] = r[j].first;
                m.w[m.n_tok] = r[j].second;
                ++m.n_tok;
            }
            miss.push_back(m);
        }
    }
    return miss;
}

}  // namespace

extern "C" {

int ref_have_avx512() { return have_avx512() ? 1 : 0; }
int ref_physical_cpus() { return int(physical_cpus().size()); }
float ref_fp16_to_fp32(uint16_t h) { return fp16_to_fp32(h); }
uint16_t ref_fp32_to_fp16(float f) { return fp32_to_fp16(f); }
size_t ref_mat_bytes(int rows, int cols) { return mat_bytes(rows, cols); }
size_t ref_expert_bytes(int n, int ff) { return expert_bytes(ExpertShape{n, ff}); }

void ref_repack(const void* ggml_rows, int rows, int cols, void* dst) { repack(ggml_rows, rows, cols, dst); }
void ref_repack_expert(const void* gate, const void* up, const void* down, int n, int ff, void* blob) {
    repack_expert(gate, up, down, ExpertShape{n, ff}, blob);
}

// Q8 of one vector: q [n], d [n/32]
void ref_quantize_q8(const float* x, int n, int8_t* q, float* d) {
    Acts a(x, 1, n);
    std::memcpy(q, a.a[0].qs, size_t(n));
    std::memcpy(d, a.a[0].d, size_t(n / kQ8Block) * 4);
}

// y [r1 - r0] of one planar matrix for one token; avx != 0 takes matvec_avx512
void ref_matvec(const void* mat, int rows, int cols, const float* x, int r0, int r1, float* y, int avx) {
    Acts a(x, 1, cols);
    const Mat w = mat_view(mat, rows, cols);
    std::vector<float> full(rows, 0.0f);
    (avx ? matvec_avx512 : matvec_ref)(w, a.a.data(), 1, r0, r1, full.data(), rows);
    std::memcpy(y, full.data() + r0, size_t(r1 - r0) * 4);
}

float ref_dot_ggml(const void* ggml_row, int cols, const float* x) {
    Acts a(x, 1, cols);
    return dot_ggml(static_cast<const GgmlBlock*>(ggml_row), a.a[0]);
}

// expert_ffn for n_tok <= 4 tokens of x [n_tok][n]; out [n_tok][n]
void ref_expert_ffn(const void* blob, int n, int ff, const float* x, int n_tok, float* out, int avx) {
    const ExpertShape s{n, ff};
    Acts a(x, n_tok, n);
    std::vector<uint8_t> scratch(expert_scratch_bytes(s) + 64);
    expert_ffn(expert_view(blob, s), a.a.data(), n_tok, out, n, scratch.data(), avx != 0);
}

// One call of q2_0::moe_cpu over all routed experts of T tokens: out [T][n]. The matvec it
// uses is the reference's choice (AVX-512 VNNI when the CPU has it).
void ref_moe_cpu(const uint8_t* experts, size_t stride, int E, int n, int ff, const float* x, int T, const int32_t* ids,
                 const float* wts, int K, float* out, int workers) {
    const ExpertShape s{n, ff};
    Acts a(x, T, n);
    const std::vector<Miss> miss = build_entries(experts, stride, E, ids, wts, T, K);
    std::vector<uint8_t> scratch(moe_cpu_scratch_bytes(s, int(miss.size()), workers));
    moe_cpu(pool(workers), s, miss.data(), int(miss.size()), a.a.data(), T, out, n, scratch.data());
}

// Timed variant for the CPU baseline: `reps` calls over `n_layers` layers of experts laid out
// back to back (layer l at experts + l * layer_stride), ids/wts/x per layer; the Q8 of x and the
// entry lists are part of every call, as they are in moe_block. Returns seconds per call, averaged.
double ref_moe_cpu_timed(const uint8_t* experts, size_t stride, size_t layer_stride, int n_layers, int E, int n, int ff,
                         const float* x, int T, const int32_t* ids, const float* wts, int K, float* out, int workers,
                         int reps) {
    const ExpertShape s{n, ff};
    CpuPool& p = pool(workers);
    std::vector<uint8_t> scratch(moe_cpu_scratch_bytes(s, T * K, workers));
    const auto t0 = std::chrono::steady_clock::now();
    for (int r = 0; r < reps; ++r) {
        const int l = r % n_layers;
        Acts a(x + size_t(l) * T * n, T, n);
        const std::vector<Miss> miss =
            build_entries(experts + size_t(l) * layer_stride, stride, E, ids + size_t(l) * T * K, wts + size_t(l) * T * K, T, K);
        moe_cpu(p, s, miss.data(), int(miss.size()), a.a.data(), T, out, n, scratch.data());
    }
    const auto t1 = std::chrono::steady_clock::now();
    return std::chrono::duration<double>(t1 - t0).count() / reps;
}

// The same loop with every call timed on its own: secs [reps] receives the seconds of each call
// (for the median and the tail of the CPU baseline).
void ref_moe_cpu_times(const uint8_t* experts, size_t stride, size_t layer_stride, int n_layers, int E, int n, int ff, const float* x,
                       int T, const int32_t* ids, const float* wts, int K, float* out, int workers, int reps, double* secs) {
    const ExpertShape s{n, ff};
    CpuPool& p = pool(workers);
    std::vector<uint8_t> scratch(moe_cpu_scratch_bytes(s, T * K, workers));
    for (int r = 0; r < reps; ++r) {
        const int l = r % n_layers;
        const auto t0 = std::chrono::steady_clock::now();
        Acts a(x + size_t(l) * T * n, T, n);
        const std::vector<Miss> miss =
            build_entries(experts + size_t(l) * layer_stride, stride, E, ids + size_t(l) * T * K, wts + size_t(l) * T * K, T, K);
        moe_cpu(p, s, miss.data(), int(miss.size()), a.a.data(), T, out, n, scratch.data());
        secs[r] = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    }
}

// One planar matrix times one token on one thread, `reps` times, cycling over n_mats matrices laid
// out back to back (many matrices: the weights come from DRAM; one: from cache). The activation is
// quantized once outside the timed loop, as the reference's own micro-benchmark does. Returns
// seconds per call; y [rows] holds the last result.
double ref_matvec_timed(const uint8_t* mats, int n_mats, int rows, int cols, const float* x, float* y, int avx, int reps) {
    Acts a(x, 1, cols);
    const size_t mb = mat_bytes(rows, cols);
    const auto t0 = std::chrono::steady_clock::now();
    for (int r = 0; r < reps; ++r) {
        const Mat w = mat_view(mats + size_t(r % n_mats) * mb, rows, cols);
        (avx ? matvec_avx512 : matvec_ref)(w, a.a.data(), 1, 0, rows, y, rows);
    }
    return std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count() / reps;
}

void ref_pool_release() {
    g_pool.reset();
    g_pool_n = 0;
}

}  // extern "C"
