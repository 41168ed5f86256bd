// ggml-layout entry points of the Q2_0 expert path: the reference's gemv:: and gemm:: functions
// (kernels/cuda/ggml_gemv.h:26-65, kernels/cuda/ggml_gemm.h:27-68) for ggml type 42, as the draft
// head's MoE calls them (arch/qwen4exp/mtp.cu:631-670), and the head's Q8_0 -> Q2_0 requantizer
// (arch/qwen4exp/mtp.cu:129-215) on the device.
//
// Weights stay in ggml's own layout here: rows of 18-byte blocks {fp16 d; 16 code bytes, element j
// in byte j / 4 at bit 2 * (j % 4)}, experts back to back. Activations are ggml's Q8_1 blocks
// {fp16 d; fp16 sum; 32 int8}, rows padded to 512 values. The arithmetic is ggml's
// (third_party/ggml/src/ggml-cuda/vecdotq.cuh:728-771): per 32-value chunk an exact integer sum
// of (q - 1) * a, scaled as d2 * d8 * sumi in float; chunks are added in float.
//
// One kernel serves every entry. A block takes one work item (an expert and up to NT activation
// rows) and a run of weight rows. The rows are contiguous in memory, so a tile of them is staged
// in shared memory by one 1-D bulk (TMA) copy; a lane owns a pair of neighbouring blocks (36 bytes,
// nine conflict-free 32-bit shared-memory loads) and the activations are kept in shared memory
// transposed so that crumb p of a weight word lines up with one int8x4 word: 16 dp4a per block and
// token, no table look-ups.
#include "frx_common.cuh"

#include <mutex>

namespace frx {
namespace {

#include "frx_group.cuh"

constexpr uint32_t kTypeQ2_0 = 42;   // core/formats.hpp:11-18
constexpr int kQ81Bytes = 36;        // block_q8_1 (third_party/ggml/src/ggml-common.h:256-268)
constexpr int kRowPad = 512;         // MATRIX_ROW_PADDING (third_party/ggml/src/ggml-cuda/common.cuh:186)
constexpr int kDotThreads = 256, kDotWarps = 8;

inline int64_t padded_cols(int64_t ncols) { return (ncols + kRowPad - 1) / kRowPad * kRowPad; }
inline size_t act_row_bytes(int64_t ncols) { return size_t(padded_cols(ncols) / kQ8) * kQ81Bytes; }

// ---- Q8_1 quantizer (third_party/ggml/src/ggml-cuda/quantize.cu:54-101): per 32 values
// d = amax / 127, q = amax == 0 ? 0 : roundf(x / d); the block keeps half(d), half(sum of the inputs).
// With `u`, the input is silu(g) * u first (gemv::swiglu_q8_1, kernels/cuda/ggml_gemv.cu:98-107,
// which uses the fast exponential).
__global__ void __launch_bounds__(256) k_q8_1(const float* __restrict__ x, const float* __restrict__ u, int64_t ncols, int64_t padded,
                                              uint8_t* __restrict__ y) {
    const int64_t i0 = int64_t(blockDim.x) * blockIdx.x + threadIdx.x, t = blockIdx.y;
    if (i0 >= padded) return;   // padded is a multiple of the block
    float xi = 0.0f;
    if (i0 < ncols) {
        xi = x[t * ncols + i0];
        if (u) xi = __fmul_rn(__fdiv_rn(xi, __fadd_rn(1.0f, __expf(-xi))), u[t * ncols + i0]);
    }
    float amax = fabsf(xi), sum = xi;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        sum = __fadd_rn(sum, __shfl_xor_sync(0xffffffffu, sum, o));
    }
    const float d = __fdiv_rn(amax, 127.0f);
    uint8_t* blk = y + (t * (padded / kQ8) + i0 / kQ8) * kQ81Bytes;
    const int iqs = int(i0 % kQ8);
    blk[4 + iqs] = uint8_t(int8_t(amax == 0.0f ? 0 : int(round_half_away(__fdiv_rn(xi, d)))));
    if (iqs == 0) *reinterpret_cast<__half2*>(blk) = __halves2half2(__float2half_rn(d), __float2half_rn(sum));
}

// ---- the dot-product kernel
struct DotArgs {
    const uint8_t* w;          // expert e's matrix at w + e * expert_stride
    const uint8_t* gate;       // fused SwiGLU: the gate matrix, same strides (or null)
    size_t expert_stride;
    const uint8_t* xq;         // Q8_1 rows
    size_t act_row;            // bytes per activation row
    float* dst;                // [rows of slots][nrows]
    int ncols, nrows;
    int rows_per_tile;         // weight rows staged per step
    int tma;                   // 1: tiles are fetched by bulk copies (alignment checked on the host)
    unsigned long long wait_ns;
    // direct jobs (gemv): job j has expert ids[j] (0 without ids), activation row j / act_div, output row j
    const int32_t* ids;
    int n_jobs, act_div;
    // grouped jobs (gemm): item i = up to NT slots of one expert from the grouped order
    const int* bounds;
    const int* item_off;
    const int32_t* perm;
    int* status;               // [1] = number of items
    int E, K, x_per_slot;
};

struct DotSmem {
    uint32_t at, d8, sa, w, bar, abort, total;
};
__host__ __device__ inline DotSmem dot_smem(int nt, int ncols, int tile_bytes, bool gate) {
    DotSmem s{};
    const uint32_t nch = uint32_t(ncols / kQ8);
    uint32_t off = 0;
    s.at = off;
    off += uint32_t(nt) * uint32_t(ncols);
    s.d8 = off;
    off += uint32_t(nt) * nch * 4;
    s.sa = off;
    off += uint32_t(nt) * nch * 4;
    off = (off + 127u) & ~127u;
    s.w = off;
    off += uint32_t(tile_bytes) * (gate ? 2u : 1u);
    off = (off + 15u) & ~15u;
    s.bar = off;
    off += 16;
    s.abort = off;
    off += 16;
    s.total = off;
    return s;
}

// One pair of neighbouring blocks (36 bytes at a 4-byte boundary) from shared memory: the two
// scales and the eight code words.
__device__ __forceinline__ void load_pair(const uint8_t* p, float& d0, float& d1, uint32_t (&c)[8]) {
    const uint32_t* q = reinterpret_cast<const uint32_t*>(p);
    uint32_t v[9];
#pragma unroll
    for (int i = 0; i < 9; ++i) v[i] = q[i];
    d0 = __half2float(__ushort_as_half(uint16_t(v[0] & 0xffffu)));
    d1 = __half2float(__ushort_as_half(uint16_t(v[4] >> 16)));
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        c[i] = __funnelshift_r(v[i], v[i + 1], 16);   // bytes 2 + 4 i .. 5 + 4 i
        c[4 + i] = v[5 + i];                          // bytes 20 + 4 i ..
    }
}

// sum over the 32 values of one chunk of (q - 1) * a: two code words against eight transposed
// activation words, minus the sum of the activation codes
__device__ __forceinline__ int chunk_sum(uint32_t w0, uint32_t w1, const uint4& a0, const uint4& a1, int suma) {
    constexpr uint32_t M = 0x03030303u;
    int s = 0;
    s = __dp4a(int(w0 & M), int(a0.x), s);
    s = __dp4a(int((w0 >> 2) & M), int(a0.y), s);
    s = __dp4a(int((w0 >> 4) & M), int(a0.z), s);
    s = __dp4a(int((w0 >> 6) & M), int(a0.w), s);
    s = __dp4a(int(w1 & M), int(a1.x), s);
    s = __dp4a(int((w1 >> 2) & M), int(a1.y), s);
    s = __dp4a(int((w1 >> 4) & M), int(a1.z), s);
    s = __dp4a(int((w1 >> 6) & M), int(a1.w), s);
    return s - suma;
}

template <int NT, bool GATE>
__global__ void __launch_bounds__(kDotThreads) k_ggml_dot(const DotArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int nb = a.ncols / kQK, np = nb / 2, nch = a.ncols / kQ8;
    const uint32_t row_bytes = uint32_t(nb) * kBlockBytes;
    const uint32_t tile_bytes = uint32_t(a.rows_per_tile) * row_bytes;
    const DotSmem sm = dot_smem(NT, a.ncols, int(tile_bytes), GATE);
    uint64_t* bar = reinterpret_cast<uint64_t*>(smem + sm.bar);
    volatile int* abort = reinterpret_cast<volatile int*>(smem + sm.abort);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    // ---- this block's work item
    __shared__ int s_act_rows[NT];
    int e = 0, m = 1;
    int act_rows[NT], dst_rows[NT];
    if (a.perm) {
        const int i = blockIdx.x;
        if (i >= a.status[1]) return;
        int lo = 0, hi = a.E;   // the expert with item_off[e] <= i < item_off[e + 1]
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (a.item_off[mid] <= i) lo = mid; else hi = mid;
        }
        e = lo;
        const int base = a.bounds[e] + (i - a.item_off[e]) * kTokPerItem;
        m = min(min(kTokPerItem, NT), a.bounds[e + 1] - base);
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            const int slot = j < m ? a.perm[base + j] : 0;
            dst_rows[j] = slot;
            act_rows[j] = a.x_per_slot ? slot : slot / a.K;
        }
    } else {
        const int j = blockIdx.x;
        e = a.ids ? a.ids[j] : 0;
#pragma unroll
        for (int q = 0; q < NT; ++q) {
            dst_rows[q] = j;
            act_rows[q] = j / a.act_div;
        }
    }
    if (tid == 0) {
        mbar_init(bar, 1);
        *abort = 0;
        mbar_fence_init();
#pragma unroll
        for (int j = 0; j < NT; ++j) s_act_rows[j] = act_rows[j];
    }
    __syncthreads();

    // ---- activations: codes transposed per 16 values (word p of a group = values p, 4 + p, 8 + p,
    // 12 + p), chunk scales, chunk code sums
    uint32_t* at = reinterpret_cast<uint32_t*>(smem + sm.at);
    float* d8 = reinterpret_cast<float*>(smem + sm.d8);
    int* sa = reinterpret_cast<int*>(smem + sm.sa);
    for (int idx = tid; idx < m * nch; idx += kDotThreads) {
        const int j = idx / nch, c = idx % nch;
        const uint32_t* blk = reinterpret_cast<const uint32_t*>(a.xq + size_t(s_act_rows[j]) * a.act_row + size_t(c) * kQ81Bytes);
        uint32_t v[9];
#pragma unroll
        for (int i = 0; i < 9; ++i) v[i] = blk[i];
        d8[j * nch + c] = __half2float(__ushort_as_half(uint16_t(v[0] & 0xffffu)));
        int s = 0;
#pragma unroll
        for (int i = 1; i < 9; ++i) s = __dp4a(int(v[i]), 0x01010101, s);
        sa[j * nch + c] = s;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint32_t u0 = v[1 + 4 * h], u1 = v[2 + 4 * h], u2 = v[3 + 4 * h], u3 = v[4 + 4 * h];
            const uint32_t lo01 = __byte_perm(u0, u1, 0x5140), hi01 = __byte_perm(u0, u1, 0x7362);
            const uint32_t lo23 = __byte_perm(u2, u3, 0x5140), hi23 = __byte_perm(u2, u3, 0x7362);
            uint4 o;
            o.x = __byte_perm(lo01, lo23, 0x5410);
            o.y = __byte_perm(lo01, lo23, 0x7632);
            o.z = __byte_perm(hi01, hi23, 0x5410);
            o.w = __byte_perm(hi01, hi23, 0x7632);
            reinterpret_cast<uint4*>(at + size_t(j) * (a.ncols / 4))[c * 2 + h] = o;
        }
    }
    __syncthreads();

    // ---- lanes: a lane owns block pairs lane_p, lane_p + stride, ... of row lane_row of a pass
    const int rpp = (np < 32 && 32 % np == 0) ? 32 / np : 1;   // rows per pass of a warp
    const int width = 32 / rpp;                                // lanes per row
    const int lane_row = lane / width, lane_p = lane % width;
    const uint8_t* wsrc = a.w + size_t(e) * a.expert_stride;
    const uint8_t* gsrc = GATE ? a.gate + size_t(e) * a.expert_stride : nullptr;
    uint8_t* wt = smem + sm.w;
    uint8_t* gt = wt + tile_bytes;
    const int n_tiles = (a.nrows + a.rows_per_tile - 1) / a.rows_per_tile;
    uint32_t phase = 0;
    for (int tile = blockIdx.y; tile < n_tiles; tile += gridDim.y) {
        const int r0 = tile * a.rows_per_tile, rows = min(a.rows_per_tile, a.nrows - r0);
        const uint32_t bytes = uint32_t(rows) * row_bytes;
        __syncthreads();   // everyone is done with the previous tile
        if (a.tma && rows == a.rows_per_tile) {
            if (tid == 0) {
                mbar_expect_tx(bar, bytes * (GATE ? 2u : 1u));
                bulk_g2s(wt, wsrc + size_t(r0) * row_bytes, bytes, bar);
                if (GATE) bulk_g2s(gt, gsrc + size_t(r0) * row_bytes, bytes, bar);
            }
            mbar_wait_bounded(bar, phase, abort, a.wait_ns);
            phase ^= 1u;
        } else {
            const uint32_t* s0 = reinterpret_cast<const uint32_t*>(wsrc + size_t(r0) * row_bytes);
            for (uint32_t i = tid; i < bytes / 4; i += kDotThreads) reinterpret_cast<uint32_t*>(wt)[i] = s0[i];
            if (GATE) {
                const uint32_t* s1 = reinterpret_cast<const uint32_t*>(gsrc + size_t(r0) * row_bytes);
                for (uint32_t i = tid; i < bytes / 4; i += kDotThreads) reinterpret_cast<uint32_t*>(gt)[i] = s1[i];
            }
            __syncthreads();
        }
        for (int rb = warp * rpp; rb < rows; rb += kDotWarps * rpp) {   // uniform for the warp: the sums below are shuffled
            const int rr = rb + lane_row;
            const bool live = rr < rows;
            float acc[NT], gacc[NT];
#pragma unroll
            for (int j = 0; j < NT; ++j) acc[j] = gacc[j] = 0.0f;
            for (int pi = lane_p; live && pi < np; pi += width) {
                float d0, d1, g0 = 0.0f, g1 = 0.0f;
                uint32_t c[8], gc[8];
                load_pair(wt + size_t(rr) * row_bytes + size_t(pi) * 36, d0, d1, c);
                if (GATE) load_pair(gt + size_t(rr) * row_bytes + size_t(pi) * 36, g0, g1, gc);
#pragma unroll
                for (int j = 0; j < NT; ++j) {
                    if (j < m) {
                        const uint4* aj = reinterpret_cast<const uint4*>(at + size_t(j) * (a.ncols / 4)) + pi * 8;
                        const float* dj = d8 + j * nch + pi * 4;
                        const int* sj = sa + j * nch + pi * 4;
#pragma unroll
                        for (int q = 0; q < 4; ++q) {   // the four chunks of the pair
                            const uint4 a0 = aj[2 * q], a1 = aj[2 * q + 1];
                            const float dw = q < 2 ? d0 : d1;
                            const int s = chunk_sum(c[2 * q], c[2 * q + 1], a0, a1, sj[q]);
                            acc[j] = __fadd_rn(acc[j], __fmul_rn(__fmul_rn(dw, dj[q]), float(s)));   // d2 * d8 * sumi
                            if (GATE) {
                                const float dg = q < 2 ? g0 : g1;
                                const int sg = chunk_sum(gc[2 * q], gc[2 * q + 1], a0, a1, sj[q]);
                                gacc[j] = __fadd_rn(gacc[j], __fmul_rn(__fmul_rn(dg, dj[q]), float(sg)));
                            }
                        }
                    }
                }
            }
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                float v = acc[j], g = gacc[j];
                for (int o = width >> 1; o > 0; o >>= 1) {
                    v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, o));
                    if (GATE) g = __fadd_rn(g, __shfl_xor_sync(0xffffffffu, g, o));
                }
                if (j < m && lane_p == 0 && live) {
                    if (GATE) v = __fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, expf(-g))), v);   // ggml unary.cuh:98-100
                    a.dst[size_t(dst_rows[j]) * a.nrows + r0 + rr] = v;
                }
            }
        }
    }
    if (*abort && tid == 0 && a.status) a.status[0] = kDevWaitTimeout;
}

int dot_tile_rows(int ncols) {
    const int np = ncols / 128;
    const int rpp = (np < 32 && 32 % np == 0) ? 32 / np : 1;
    return kDotWarps * rpp * 2;   // two passes of every warp per tile: 18 KB of weights at the usual shapes
}

template <int NT, bool GATE>
int launch_dot(DotArgs a, int grid_x, cudaStream_t stream) {
    a.rows_per_tile = dot_tile_rows(a.ncols);
    const uint32_t row_bytes = uint32_t(a.ncols / kQK) * kBlockBytes, tile_bytes = uint32_t(a.rows_per_tile) * row_bytes;
    a.tma = ((uintptr_t(a.w) | uintptr_t(a.gate) | a.expert_stride | tile_bytes) % 16 == 0) ? 1 : 0;
    a.wait_ns = wait_limit_ns();
    const DotSmem sm = dot_smem(NT, a.ncols, int(tile_bytes), GATE);
    if (int(sm.total) > max_smem_optin() - 1024) return fail(FRX_ERR_SHAPE, "ggml-layout product: ncols %d needs %u bytes of shared memory", a.ncols, sm.total);
    static std::mutex mu;
    static unsigned set_mask[64] = {};
    int dev = 0;
    FRX_CUDA(cudaGetDevice(&dev));
    {
        std::lock_guard<std::mutex> lk(mu);
        const unsigned bit = 1u << ((NT > 1 ? 2 : 0) + (GATE ? 1 : 0));
        if (dev >= 0 && dev < 64 && !(set_mask[dev] & bit)) {
            FRX_CUDA(cudaFuncSetAttribute(k_ggml_dot<NT, GATE>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem_optin() - 1024));   // less the static part
            set_mask[dev] |= bit;
        }
    }
    const int n_tiles = (a.nrows + a.rows_per_tile - 1) / a.rows_per_tile;
    // enough blocks to fill the GPU, each walking several tiles so the activation set-up is amortised
    const int sms = sm_count() > 0 ? sm_count() : 148;
    int gy = n_tiles;
    while (gy > 1 && (long long)grid_x * gy > 8LL * sms && gy % 2 == 0) gy /= 2;
    k_ggml_dot<NT, GATE><<<dim3(unsigned(grid_x), unsigned(gy)), kDotThreads, sm.total, stream>>>(a);
    FRX_CUDA(cudaGetLastError());
    return FRX_OK;
}

int check_dot_shape(const char* who, uint32_t type, int64_t ncols, int64_t nrows) {
    if (type != kTypeQ2_0) return fail(FRX_ERR_SHAPE, "%s: ggml type %u is not built (only Q2_0, type 42)", who, type);
    if (ncols < 128 || ncols % 128 || ncols > 16384 || nrows < 1 || nrows > (1 << 24))
        return fail(FRX_ERR_SHAPE, "%s: ncols %lld must be a multiple of 128 (at most 16384), nrows %lld positive", who, (long long)ncols,
                    (long long)nrows);
    return FRX_OK;
}

// ---- Q8_0 -> Q2_0 (arch/qwen4exp/mtp.cu:129-201): one warp per 64 values. Lane l holds values l
// and 32 + l; lanes 0..23 each try one candidate scale, adding the squared errors in index order.
__device__ __forceinline__ int q2_code_dev(float v) { return int(v >= 0.5f) + int(v >= 1.5f) - int(v <= -0.5f); }
__global__ void __launch_bounds__(256) k_q8_0_to_q2_0(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, size_t nblocks64) {
    const size_t b = size_t(blockIdx.x) * 8 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (b >= nblocks64) return;
    const uint8_t* s = src + b * 68;
    const float d_lo = __half2float(__ushort_as_half(uint16_t(s[0] | (s[1] << 8))));
    const float d_hi = __half2float(__ushort_as_half(uint16_t(s[34] | (s[35] << 8))));
    const float x_lo = __fmul_rn(d_lo, float(int8_t(s[2 + lane]))), x_hi = __fmul_rn(d_hi, float(int8_t(s[36 + lane])));
    float amax = fmaxf(fabsf(x_lo), fabsf(x_hi));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    // candidate `lane`: d = amax / (2.5f - 1.5f * float(c) / 23.0f), through fp16
    const float div = __fsub_rn(2.5f, __fdiv_rn(__fmul_rn(1.5f, float(lane)), 23.0f));
    const float dq = __half2float(__float2half_rn(__fdiv_rn(amax, div)));
    const bool usable = dq > 0.0f && dq < INFINITY;   // else every code is 0 (see the oracle's note on lround)
    float e = 0.0f;
    for (int j = 0; j < 64; ++j) {
        const float xj = __shfl_sync(0xffffffffu, j < 32 ? x_lo : x_hi, j & 31);
        const int q = usable ? q2_code_dev(__fdiv_rn(xj, dq)) : 0;
        const float r = __fsub_rn(xj, __fmul_rn(float(q), dq));
        e = __fadd_rn(e, __fmul_rn(r, r));
    }
    // the first candidate with the smallest error wins; a NaN or infinite error never does
    bool ok = lane < 24 && amax > 0.0f && e < INFINITY;
    float be = ok ? e : INFINITY, bd = ok ? dq : 0.0f;
    int bc = ok ? lane : 64;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float oe = __shfl_xor_sync(0xffffffffu, be, o), od = __shfl_xor_sync(0xffffffffu, bd, o);
        const int oc = __shfl_xor_sync(0xffffffffu, bc, o);
        if (oc < 64 && (bc == 64 || oe < be || (oe == be && oc < bc))) {
            be = oe;
            bd = od;
            bc = oc;
        }
    }
    const float best_d = bc < 64 ? bd : 0.0f;
    const bool fin = best_d > 0.0f && best_d < INFINITY;
    const int c_lo = best_d > 0.0f ? (fin ? q2_code_dev(__fdiv_rn(x_lo, best_d)) : 0) + 1 : 1;
    const int c_hi = best_d > 0.0f ? (fin ? q2_code_dev(__fdiv_rn(x_hi, best_d)) : 0) + 1 : 1;
    // byte L (L < 16) holds elements 4 L .. 4 L + 3
    uint32_t byte = 0;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int srcl = (4 * lane + k) & 31;
        const int v_lo = __shfl_sync(0xffffffffu, c_lo, srcl), v_hi = __shfl_sync(0xffffffffu, c_hi, srcl);
        byte |= uint32_t(lane < 8 ? v_lo : v_hi) << (2 * k);
    }
    uint8_t* o = dst + b * 18;
    if (lane < 16) o[2 + lane] = uint8_t(byte);
    if (lane == 0) *reinterpret_cast<__half*>(o) = __float2half_rn(best_d);   // blocks are 18 bytes: the scale is 2-byte aligned
}

// ---- grouped plan in a workspace
struct PlanLayout {
    size_t status, chunk_cnt, bounds, item_off, perm, act, total;
    int n_chunks, max_items;
};
PlanLayout plan_layout(int64_t ncols, int64_t rows, int E) {
    PlanLayout L{};
    size_t off = 0;
    auto take = [&](size_t bytes) {
        const size_t o = off;
        off += align_up(bytes);
        return o;
    };
    L.n_chunks = int((rows + kChunkSlots - 1) / kChunkSlots);
    L.max_items = int(rows / kTokPerItem) + E;
    L.status = take(64);
    L.chunk_cnt = take(size_t(L.n_chunks) * E * 4);
    L.bounds = take(size_t(E + 1) * 4);
    L.item_off = take(size_t(E + 1) * 4);
    L.perm = take(size_t(rows) * 4);
    L.act = take(size_t(rows) * act_row_bytes(ncols));
    L.total = off;
    return L;
}
constexpr int kPlanMaxExperts = 4096;

}  // namespace
}  // namespace frx

using namespace frx;

extern "C" {

size_t frx_gemv_q8_1_bytes(int64_t ncols, int n_tok) {
    if (ncols < 1 || n_tok < 1) return 0;
    return size_t(n_tok) * act_row_bytes(ncols);
}

int64_t frx_gemv_row_bytes(uint32_t ggml_type, int64_t ncols) {
    if (ggml_type != kTypeQ2_0 || ncols < 0) return 0;
    return ncols / kQK * kBlockBytes;
}

int frx_gemv_quantize_q8_1(const float* x, int64_t ncols, int n_tok, void* xq, frx_stream_t stream) {
    if (ncols < 1 || n_tok < 0) return fail(FRX_ERR_SHAPE, "gemv::quantize_q8_1: ncols %lld, n_tok %d", (long long)ncols, n_tok);
    if (n_tok == 0) return FRX_OK;
    if (!x || !xq || uintptr_t(xq) % 4) return fail(FRX_ERR_ARG, "gemv::quantize_q8_1: null or misaligned pointer");
    const int64_t padded = padded_cols(ncols);
    FRX_LAUNCH(kKQuant, stream, k_q8_1<<<dim3(unsigned(padded / 256), unsigned(n_tok)), 256, 0, stream>>>(x, nullptr, ncols, padded, static_cast<uint8_t*>(xq)));
    FRX_CUDA(cudaGetLastError());
    return FRX_OK;
}

int frx_gemv_swiglu_q8_1(const float* g, const float* u, int64_t ncols, int n_tok, void* xq, frx_stream_t stream) {
    if (ncols < 1 || n_tok < 0) return fail(FRX_ERR_SHAPE, "gemv::swiglu_q8_1: ncols %lld, n_tok %d", (long long)ncols, n_tok);
    if (n_tok == 0) return FRX_OK;
    if (!g || !u || !xq || uintptr_t(xq) % 4) return fail(FRX_ERR_ARG, "gemv::swiglu_q8_1: null or misaligned pointer");
    const int64_t padded = padded_cols(ncols);
    FRX_LAUNCH(kKQuant, stream, k_q8_1<<<dim3(unsigned(padded / 256), unsigned(n_tok)), 256, 0, stream>>>(g, u, ncols, padded, static_cast<uint8_t*>(xq)));
    FRX_CUDA(cudaGetLastError());
    return FRX_OK;
}

int frx_gemv_moe_q(uint32_t ggml_type, const void* w, const void* gate, const void* xq, const int32_t* ids, float* dst, int n_tok, int k,
                   int64_t ncols, int64_t nrows, int64_t expert_stride_bytes, int act_per_expert, frx_stream_t stream) {
    if (int rc = check_dot_shape("gemv::moe_q", ggml_type, ncols, nrows)) return rc;
    if (n_tok < 1 || n_tok > 8 || k < 1) return fail(FRX_ERR_SHAPE, "gemv::moe_q: n_tok %d must be 1..8, k %d positive", n_tok, k);
    if (!w || !xq || !ids || !dst) return fail(FRX_ERR_ARG, "gemv::moe_q: null pointer");
    if (expert_stride_bytes < 0 || expert_stride_bytes % kBlockBytes || (uintptr_t(w) | uintptr_t(gate) | uintptr_t(xq)) % 4 || expert_stride_bytes % 4)
        return fail(FRX_ERR_ARG, "gemv::moe_q: the expert stride must be whole blocks and, like the pointers, a multiple of 4 bytes");
    DotArgs a{};
    a.w = static_cast<const uint8_t*>(w);
    a.gate = static_cast<const uint8_t*>(gate);
    a.expert_stride = size_t(expert_stride_bytes);
    a.xq = static_cast<const uint8_t*>(xq);
    a.act_row = act_row_bytes(ncols);
    a.dst = dst;
    a.ncols = int(ncols);
    a.nrows = int(nrows);
    a.ids = ids;
    a.n_jobs = n_tok * k;
    a.act_div = act_per_expert ? 1 : k;
    if (gate)
        FRX_LAUNCH(kKGateUp, stream, { if (int rc = launch_dot<1, true>(a, a.n_jobs, stream)) return rc; });
    else
        FRX_LAUNCH(kKDown, stream, { if (int rc = launch_dot<1, false>(a, a.n_jobs, stream)) return rc; });
    return FRX_OK;
}

int frx_gemv_moe_q2_0(const void* w, const void* gate, const void* xq, const int32_t* ids, float* dst, int n_ids, int64_t ncols,
                      int64_t nrows, int64_t slot_stride_bytes, int per_channel_act, frx_stream_t stream) {
    if (n_ids < 1) return fail(FRX_ERR_SHAPE, "gemv::moe_q2_0: n_ids %d", n_ids);
    if (int rc = check_dot_shape("gemv::moe_q2_0", kTypeQ2_0, ncols, nrows)) return rc;
    if (!w || !xq || !ids || !dst) return fail(FRX_ERR_ARG, "gemv::moe_q2_0: null pointer");
    if (slot_stride_bytes < 0 || slot_stride_bytes % kBlockBytes || (uintptr_t(w) | uintptr_t(gate) | uintptr_t(xq)) % 4 || slot_stride_bytes % 4)
        return fail(FRX_ERR_ARG, "gemv::moe_q2_0: the slot stride must be whole blocks and, like the pointers, a multiple of 4 bytes");
    DotArgs a{};
    a.w = static_cast<const uint8_t*>(w);
    a.gate = static_cast<const uint8_t*>(gate);
    a.expert_stride = size_t(slot_stride_bytes);
    a.xq = static_cast<const uint8_t*>(xq);
    a.act_row = act_row_bytes(ncols);
    a.dst = dst;
    a.ncols = int(ncols);
    a.nrows = int(nrows);
    a.ids = ids;
    a.n_jobs = n_ids;
    a.act_div = per_channel_act ? 1 : n_ids;   // one activation row for every channel, or one each
    if (gate)
        FRX_LAUNCH(kKGateUp, stream, { if (int rc = launch_dot<1, true>(a, a.n_jobs, stream)) return rc; });
    else
        FRX_LAUNCH(kKDown, stream, { if (int rc = launch_dot<1, false>(a, a.n_jobs, stream)) return rc; });
    return FRX_OK;
}

int frx_gemv_matvec_q(uint32_t ggml_type, const void* W, const void* xq, float* y, int64_t ncols, int64_t nrows, int n_tok,
                      frx_stream_t stream) {
    if (int rc = check_dot_shape("gemv::matvec_q", ggml_type, ncols, nrows)) return rc;
    if (n_tok < 1 || n_tok > 8) return fail(FRX_ERR_SHAPE, "gemv::matvec_q: n_tok %d must be 1..8", n_tok);
    if (!W || !xq || !y || (uintptr_t(W) | uintptr_t(xq)) % 4) return fail(FRX_ERR_ARG, "gemv::matvec_q: null or misaligned pointer");
    DotArgs a{};
    a.w = static_cast<const uint8_t*>(W);
    a.expert_stride = 0;
    a.xq = static_cast<const uint8_t*>(xq);
    a.act_row = act_row_bytes(ncols);
    a.dst = y;
    a.ncols = int(ncols);
    a.nrows = int(nrows);
    a.n_jobs = n_tok;
    a.act_div = 1;
    FRX_LAUNCH(kKDown, stream, { if (int rc = launch_dot<1, false>(a, a.n_jobs, stream)) return rc; });
    return FRX_OK;
}

int frx_gemv_matvec(uint32_t ggml_type, const void* W, const float* x, float* y, int64_t ncols, int64_t nrows, int n_tok, void* scratch,
                    frx_stream_t stream) {
    if (int rc = check_dot_shape("gemv::matvec", ggml_type, ncols, nrows)) return rc;
    if (!scratch) return fail(FRX_ERR_ARG, "gemv::matvec: null scratch");
    if (int rc = frx_gemv_quantize_q8_1(x, ncols, n_tok, scratch, stream)) return rc;
    return frx_gemv_matvec_q(ggml_type, W, scratch, y, ncols, nrows, n_tok, stream);
}

size_t frx_gemm_workspace_bytes(int64_t ncols, int64_t rows) {
    if (ncols < 1 || rows < 1) return 0;
    return plan_layout(ncols, rows, kPlanMaxExperts).total;
}

int frx_gemm_moe_prepare(frx_gemm_moe_plan* plan, uint32_t ggml_type, int n_experts, const float* x, int x_per_slot, const int32_t* ids,
                         int64_t T, int K, int64_t ncols, void* ws, size_t ws_bytes, frx_stream_t stream) {
    if (!plan) return fail(FRX_ERR_ARG, "gemm::moe_prepare: null plan");
    if (int rc = check_dot_shape("gemm::moe_prepare", ggml_type, ncols, 1)) return rc;
    if (n_experts < 1 || n_experts > kPlanMaxExperts || K < 1 || T < 0 || T * K > (int64_t(1) << 28))
        return fail(FRX_ERR_SHAPE, "gemm::moe_prepare: unsupported E %d, K %d, T %lld", n_experts, K, (long long)T);
    if (!x || !ids || !ws || uintptr_t(ws) % kAlign) return fail(FRX_ERR_ARG, "gemm::moe_prepare: null pointer or workspace not 256-byte aligned");
    const int64_t rows = T * K;
    plan->type = ggml_type;
    plan->n_experts = n_experts;
    plan->K = K;
    plan->T = T;
    plan->ncols = ncols;
    plan->rows = rows;
    plan->x_per_slot = x_per_slot ? 1 : 0;
    plan->ws = ws;
    if (T == 0) return FRX_OK;
    const PlanLayout L = plan_layout(ncols, rows, n_experts);
    if (ws_bytes < L.total) return fail(FRX_ERR_WORKSPACE, "gemm::moe_prepare: workspace %zu < %zu", ws_bytes, L.total);
    auto* base = static_cast<uint8_t*>(ws);
    int* status = reinterpret_cast<int*>(base + L.status);
    int* chunk_cnt = reinterpret_cast<int*>(base + L.chunk_cnt);
    int* bounds = reinterpret_cast<int*>(base + L.bounds);
    int* item_off = reinterpret_cast<int*>(base + L.item_off);
    int32_t* perm = reinterpret_cast<int32_t*>(base + L.perm);
    const int S = int(rows), E = n_experts;
    // one Q8_1 row per token, or per (token, expert) slot when every slot has its own activations
    if (int rc = frx_gemv_quantize_q8_1(x, ncols, int(x_per_slot ? rows : T), base + L.act, stream)) return rc;
    FRX_LAUNCH(kKGroup, stream, k_pf_hist<<<L.n_chunks, 256, size_t(E) * 4, stream>>>(ids, S, E, chunk_cnt, status));
    FRX_LAUNCH(kKGroup, stream, k_pf_scan<<<1, 1024, 0, stream>>>(chunk_cnt, L.n_chunks, E, bounds, item_off, status, L.max_items));
    FRX_LAUNCH(kKGroup, stream, k_pf_place<<<L.n_chunks, 32, size_t(E) * 4, stream>>>(ids, S, E, chunk_cnt, bounds, perm));
    FRX_CUDA(cudaGetLastError());
    return FRX_OK;
}

int frx_gemm_moe_run(const frx_gemm_moe_plan* plan, const void* W, int64_t expert_stride_bytes, float* y, int64_t nrows, frx_stream_t stream) {
    if (!plan || !plan->ws) return fail(FRX_ERR_ARG, "gemm::moe_run: no plan");
    if (int rc = check_dot_shape("gemm::moe_run", plan->type, plan->ncols, nrows)) return rc;
    if (!W || !y) return fail(FRX_ERR_ARG, "gemm::moe_run: null pointer");
    if (expert_stride_bytes < 0 || expert_stride_bytes % kBlockBytes || uintptr_t(W) % 4 || expert_stride_bytes % 4)
        return fail(FRX_ERR_ARG, "gemm::moe_run: the expert stride must be whole blocks and, like W, a multiple of 4 bytes");
    if (plan->T == 0) return FRX_OK;
    const PlanLayout L = plan_layout(plan->ncols, plan->rows, plan->n_experts);
    auto* base = static_cast<uint8_t*>(plan->ws);
    DotArgs a{};
    a.w = static_cast<const uint8_t*>(W);
    a.expert_stride = size_t(expert_stride_bytes);
    a.xq = base + L.act;
    a.act_row = act_row_bytes(plan->ncols);
    a.dst = y;
    a.ncols = int(plan->ncols);
    a.nrows = int(nrows);
    a.bounds = reinterpret_cast<const int*>(base + L.bounds);
    a.item_off = reinterpret_cast<const int*>(base + L.item_off);
    a.perm = reinterpret_cast<const int32_t*>(base + L.perm);
    a.status = reinterpret_cast<int*>(base + L.status);
    a.E = plan->n_experts;
    a.K = plan->K;
    a.x_per_slot = plan->x_per_slot;
    FRX_LAUNCH(kKDown, stream, { if (int rc = launch_dot<kTokPerItem, false>(a, L.max_items, stream)) return rc; });
    return FRX_OK;
}

int frx_gemm_moe(uint32_t ggml_type, const void* W, int64_t expert_stride_bytes, int n_experts, const float* x, int x_per_slot,
                 const int32_t* ids, int64_t T, int K, float* y, int64_t ncols, int64_t nrows, void* ws, size_t ws_bytes, frx_stream_t stream) {
    frx_gemm_moe_plan plan;
    if (int rc = frx_gemm_moe_prepare(&plan, ggml_type, n_experts, x, x_per_slot, ids, T, K, ncols, ws, ws_bytes, stream)) return rc;
    return frx_gemm_moe_run(&plan, W, expert_stride_bytes, y, nrows, stream);
}

int frx_convert_q8_0_to_q2_0(const void* src_q8_0, void* dst_q2_0, size_t nblocks64, frx_stream_t stream) {
    if (nblocks64 == 0) return FRX_OK;
    if (!src_q8_0 || !dst_q2_0) return fail(FRX_ERR_ARG, "convert_q8_0_to_q2_0: null pointer");
    if (nblocks64 > (size_t(1) << 34)) return fail(FRX_ERR_SHAPE, "convert_q8_0_to_q2_0: too many blocks");
    FRX_LAUNCH(kKLayout, stream, k_q8_0_to_q2_0<<<unsigned((nblocks64 + 7) / 8), 256, 0, stream>>>(static_cast<const uint8_t*>(src_q8_0), static_cast<uint8_t*>(dst_q2_0), nblocks64));
    FRX_CUDA(cudaGetLastError());
    return FRX_OK;
}

}  // extern "C"
