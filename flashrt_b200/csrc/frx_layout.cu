// Q2_0 storage on the device: ggml -> planar repack, planar <-> tiled relayout, dequantisation.
// All three are pure permutations or element-wise decodes, so they are bit-exact by construction;
// the tests check them against the CPU oracle byte for byte.
#include "frx_common.cuh"

namespace frx {
namespace {

// ---- q2_0::repack (quant/q2_0/q2_0.cpp:34-39,51-62): one thread per output 32-bit word.
// Planar word w of a block (bytes 4w..4w+3) takes, for g = 0..3, the four 2-bit fields of ggml
// code byte 4g + w and puts them at bit 2g of its four bytes.
__global__ void k_repack(const uint8_t* __restrict__ ggml, size_t nblk, uint8_t* __restrict__ planar) {
    const size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x;   // (block, word)
    if (i >= nblk * 4) return;
    const size_t blk = i >> 2;
    const int w = int(i & 3);
    const uint8_t* b = ggml + blk * kBlockBytes;
    uint32_t out = 0;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
        const uint32_t byte = b[2 + 4 * g + w];
        const uint32_t spread = (byte & 3u) | ((byte >> 2) & 3u) << 8 | ((byte >> 4) & 3u) << 16 | ((byte >> 6) & 3u) << 24;
        out |= spread << (2 * g);
    }
    reinterpret_cast<uint32_t*>(planar)[i] = out;
    if (w == 0) reinterpret_cast<uint16_t*>(planar + nblk * 16)[blk] = uint16_t(b[0]) | uint16_t(b[1]) << 8;
}

// Geometry of one tiled expert.
struct Geo {
    int n, ff;
    int gu_groups, gu_units;   // ff/8 groups of n/128 units
    int dn_groups, dn_units;   // n/16 groups of ff/128 units
    size_t gu_mat;             // bytes of one planar gate/up matrix
    __host__ __device__ Geo(int n_, int ff_)
        : n(n_), ff(ff_), gu_groups(ff_ / 8), gu_units(n_ / kUnitK), dn_groups(n_ / 16), dn_units(ff_ / kUnitK),
          gu_mat(size_t(ff_) * (n_ / kQK) * kBlockBytes) {}
    __host__ __device__ size_t total_units() const { return size_t(gu_groups) * gu_units + size_t(dn_groups) * dn_units; }
};

// For unit `unit` of an expert and M row m: the planar matrix offset, its row count, blocks per
// row, and the matrix row that M row m is.
__device__ __forceinline__ void unit_source(const Geo& G, size_t unit, int m, size_t& mat_off, int& rows, int& nb, int& row,
                                            int& u) {
    const size_t gu_total = size_t(G.gu_groups) * G.gu_units;
    if (unit < gu_total) {
        const int grp = int(unit / G.gu_units);
        u = int(unit % G.gu_units);
        mat_off = m < 8 ? 0 : G.gu_mat;   // gate, then up
        rows = G.ff;
        nb = G.n / kQK;
        row = grp * 8 + (m & 7);
    } else {
        const size_t k = unit - gu_total;
        const int grp = int(k / G.dn_units);
        u = int(k % G.dn_units);
        mat_off = 2 * G.gu_mat;
        rows = G.n;
        nb = G.ff / kQK;
        row = grp * 16 + m;
    }
}

// One thread per 32-bit word of a unit: 128 code words, then 16 scale words (two fp16 each).
// TO_TILED: planar -> tiled; otherwise tiled -> planar.
template <bool TO_TILED>
__global__ void k_tile(const uint8_t* __restrict__ src, size_t src_stride, uint8_t* __restrict__ dst, size_t dst_stride, int n,
                       int ff, size_t units_per_expert, size_t total_words) {
    const size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= total_words) return;
    const Geo G(n, ff);
    constexpr int kWordsPerUnit = kUnitBytes / 4;   // 144
    const size_t unit_global = i / kWordsPerUnit;
    const int w = int(i % kWordsPerUnit);
    const size_t e = unit_global / units_per_expert, unit = unit_global % units_per_expert;
    const uint8_t* planar = (TO_TILED ? src + e * src_stride : nullptr);
    uint8_t* planar_out = (TO_TILED ? nullptr : dst + e * dst_stride);
    const size_t tiled_off = unit * kUnitBytes + size_t(w) * 4;
    size_t mat_off;
    int rows, nb, row, u;
    if (w < 128) {   // codes: lane L = w / 4, word (h, j) = w % 4
        const int L = w >> 2, h = (w >> 1) & 1, j = w & 1, g = L >> 2, t = L & 3;
        unit_source(G, unit, g + 8 * h, mat_off, rows, nb, row, u);
        const size_t p_off = mat_off + (size_t(row) * nb + (2 * u + j)) * 16 + size_t(t) * 4;
        if (TO_TILED)
            *reinterpret_cast<uint32_t*>(dst + e * dst_stride + tiled_off) = *reinterpret_cast<const uint32_t*>(planar + p_off);
        else
            *reinterpret_cast<uint32_t*>(planar_out + p_off) = *reinterpret_cast<const uint32_t*>(src + e * src_stride + tiled_off);
    } else {         // scales: word s = w - 128 holds [g][h][j = 0, 1], g = s / 2, h = s % 2
        const int s = w - 128, g = s >> 1, h = s & 1;
        unit_source(G, unit, g + 8 * h, mat_off, rows, nb, row, u);
        const size_t p_off = mat_off + size_t(rows) * nb * 16 + (size_t(row) * nb + 2 * u) * 2;   // two adjacent blocks
        if (TO_TILED)
            *reinterpret_cast<uint32_t*>(dst + e * dst_stride + tiled_off) = *reinterpret_cast<const uint32_t*>(planar + p_off);
        else
            *reinterpret_cast<uint32_t*>(planar_out + p_off) = *reinterpret_cast<const uint32_t*>(src + e * src_stride + tiled_off);
    }
}

// Dequantise one matrix of a tiled expert: one thread per (row, block), 64 floats out.
// which: 0 gate, 1 up, 2 down.
__global__ void k_dequant(const uint8_t* __restrict__ blob, int n, int ff, int which, float* __restrict__ out) {
    const int rows = which == 2 ? n : ff, cols = which == 2 ? ff : n, nb = cols / kQK;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows * nb) return;
    const int row = i / nb, b = i % nb, u = b >> 1, j = b & 1;
    const Geo G(n, ff);
    size_t unit;
    int m;
    if (which == 2) {
        unit = size_t(G.gu_groups) * G.gu_units + size_t(row / 16) * G.dn_units + u;
        m = row % 16;
    } else {
        unit = size_t(row / 8) * G.gu_units + u;
        m = (row % 8) + (which == 1 ? 8 : 0);
    }
    const uint8_t* up = blob + unit * kUnitBytes;
    const int g = m & 7, h = m >> 3;
    const __half d = *reinterpret_cast<const __half*>(up + kUnitCodeBytes + g * 8 + (h * 2 + j) * 2);
    const float df = __half2float(d);
    float* o = out + size_t(row) * cols + size_t(b) * kQK;
#pragma unroll
    for (int t = 0; t < 4; ++t) {
        const uint32_t word = *reinterpret_cast<const uint32_t*>(up + (g * 4 + t) * 16 + (h * 2 + j) * 4);
#pragma unroll
        for (int p = 0; p < 4; ++p)
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int q = int((word >> (8 * k + 2 * p)) & 3u);
                o[16 * p + 4 * t + k] = __fmul_rn(float(q - 1), df);
            }
    }
}

int check_shape(const char* who, int n, int ff) {
    if (n < kUnitK || ff < kUnitK || n % kUnitK || ff % kUnitK)
        return fail(FRX_ERR_SHAPE, "%s: n %d and ff %d must be positive multiples of %d", who, n, ff, kUnitK);
    return FRX_OK;
}

template <bool TO_TILED>
int tile_launch(const char* who, const void* src, size_t src_stride, void* dst, size_t dst_stride, int n_experts, int n, int ff,
                cudaStream_t stream) {
    if (!src || !dst) return fail(FRX_ERR_ARG, "%s: null pointer", who);
    if (n_experts < 0) return fail(FRX_ERR_ARG, "%s: n_experts %d", who, n_experts);
    if (int rc = check_shape(who, n, ff)) return rc;
    const size_t blob = frx_q2_expert_bytes(n, ff);
    if (src_stride < blob || dst_stride < blob || (src_stride | dst_stride) % 4 || (uintptr_t(src) | uintptr_t(dst)) % 4)
        return fail(FRX_ERR_ARG, "%s: strides %zu / %zu must be >= %zu and, like the pointers, 4-byte aligned", who, src_stride,
                    dst_stride, blob);
    if (n_experts == 0) return FRX_OK;
    const Geo G(n, ff);
    const size_t words = size_t(n_experts) * G.total_units() * (kUnitBytes / 4);
    const unsigned grid = unsigned((words + 255) / 256);
    k_tile<TO_TILED><<<grid, 256, 0, stream>>>(static_cast<const uint8_t*>(src), src_stride, static_cast<uint8_t*>(dst), dst_stride,
                                               n, ff, G.total_units(), words);
    FRX_CUDA(cudaGetLastError());
    return FRX_OK;
}

}  // namespace
}  // namespace frx

using namespace frx;

extern "C" {

int frx_q2_repack(const void* ggml_rows, int rows, int cols, void* planar, frx_stream_t stream) {
    if (!ggml_rows || !planar) return fail(FRX_ERR_ARG, "frx_q2_repack: null pointer");
    if (rows < 0 || cols < kQK || cols % kQK) return fail(FRX_ERR_SHAPE, "frx_q2_repack: rows %d, cols %d", rows, cols);
    if (uintptr_t(planar) % 4) return fail(FRX_ERR_ARG, "frx_q2_repack: planar must be 4-byte aligned");
    const size_t nblk = size_t(rows) * (cols / kQK);
    if (nblk == 0) return FRX_OK;
    k_repack<<<unsigned((nblk * 4 + 255) / 256), 256, 0, stream>>>(static_cast<const uint8_t*>(ggml_rows), nblk,
                                                                  static_cast<uint8_t*>(planar));
    FRX_CUDA(cudaGetLastError());
    return FRX_OK;
}

int frx_q2_tile_experts(const void* src_planar, size_t src_stride, void* dst_tiled, size_t dst_stride, int n_experts, int n,
                        int ff, frx_stream_t stream) {
    return tile_launch<true>("frx_q2_tile_experts", src_planar, src_stride, dst_tiled, dst_stride, n_experts, n, ff, stream);
}

int frx_q2_untile_experts(const void* src_tiled, size_t src_stride, void* dst_planar, size_t dst_stride, int n_experts, int n,
                          int ff, frx_stream_t stream) {
    return tile_launch<false>("frx_q2_untile_experts", src_tiled, src_stride, dst_planar, dst_stride, n_experts, n, ff, stream);
}

int frx_q2_dequant_expert(const void* tiled_blob, int n, int ff, float* gate, float* up, float* down, frx_stream_t stream) {
    if (!tiled_blob) return fail(FRX_ERR_ARG, "frx_q2_dequant_expert: null blob");
    if (int rc = check_shape("frx_q2_dequant_expert", n, ff)) return rc;
    if (uintptr_t(tiled_blob) % 16) return fail(FRX_ERR_ARG, "frx_q2_dequant_expert: blob must be 16-byte aligned");
    float* outs[3] = {gate, up, down};
    for (int which = 0; which < 3; ++which) {
        if (!outs[which]) continue;
        const int rows = which == 2 ? n : ff, nb = (which == 2 ? ff : n) / kQK;
        k_dequant<<<(rows * nb + 127) / 128, 128, 0, stream>>>(static_cast<const uint8_t*>(tiled_blob), n, ff, which, outs[which]);
        FRX_CUDA(cudaGetLastError());
    }
    return FRX_OK;
}

}  // extern "C"
