// Decode-sized MoE layer: quantize x, group (token, expert) slots by expert, gate/up + SwiGLU,
// down, ordered weighted combine. Experts are streamed once from HBM in the tiled layout by a
// producer warp issuing 1-D bulk (TMA) copies into a shared-memory ring; consumer warps unpack the
// 2-bit codes in registers and feed int8 tensor-core MMAs whose N dimension is the (at most 8)
// tokens routed to the expert. Integer sums are exact; the float scaling and the accumulation over
// the blocks of a row run in one lane, in block order, with the roundings of the reference's
// scalar matvec (quant/q2_0/q2_0.cpp:119-140), so results match it bit for bit.
#include "frx_common.cuh"
#include "frx_route.cuh"

#include <cuda_bf16.h>

#include <cstring>
#include <mutex>

namespace frx {
namespace {

#include "frx_group.cuh"

constexpr int kMaxChunkTokens = 64;   // tokens grouped by one k_group launch
constexpr int kNarrowTok = 4;         // items of at most this many tokens take the narrow form of the inner product (units_mma_narrow)

// One unit of expert work: a tiled expert blob and up to 8 (token, expert) slots routed to it.
// A slot is a row of the hidden and output buffers: t * K + k for the k-th expert of token t,
// TK + t for the shared expert of token t.
struct __align__(16) Item {
    const uint8_t* blob;
    int32_t n_tok;
    int32_t expert;              // for diagnostics: the expert id, -1 for the shared expert
    int32_t slot[kTokPerItem];
};
static_assert(sizeof(Item) == 48, "Item is 48 bytes");
constexpr int kItemWords = sizeof(Item) / 4;

__host__ __device__ inline int slot_token(int slot, int K, int TK) { return slot < TK ? slot / K : slot - TK; }

// Workspace status words: [0] device error, [1] items of the current chunk, [2] detail, [3] cookie.
// Behind the kStatusWords words, in the decode layout: one counter per item, the gate/up tasks of the
// item that have been finished (zeroed by the grouping kernel, counted and awaited by k_ffn).
constexpr int kStatusWords = 16;
constexpr int kMaxStreamBlocks = 1024;   // the streaming kernels run one block per SM
struct Layout {
    size_t status, ranges, items, order, xq, xa, xc, gu, h, hq, ha, hc, y, ysh, total;
    int max_items;
};

Layout make_layout(int T, int K, int n, int ff) {
    const int Tc = T < kMaxChunkTokens ? T : kMaxChunkTokens;
    Layout L{};
    size_t off = 0;
    auto take = [&](size_t bytes) {
        const size_t o = off;
        off += align_up(bytes);
        return o;
    };
    L.max_items = Tc * K + (Tc + kNarrowTok - 1) / kNarrowTok;   // every routed slot its own item at worst; the shared expert in items of four tokens
    L.status = take(64 + size_t(L.max_items) * 4);   // 16 status words, then one counter per item (see k_ffn)
    L.ranges = take((kMaxStreamBlocks + 1) * 4);   // the down kernel's tasks per block (see DownSplit)
    L.items = take(size_t(L.max_items) * sizeof(Item));
    L.order = take(size_t(Tc) * K * 4);
    L.xq = take(size_t(Tc) * n);
    L.xa = take(size_t(Tc) * (n / kQ8) * 4);
    L.xc = take(size_t(Tc) * (n / kQ8) * 4);
    L.gu = take(size_t(Tc) * (K + 1) * ff * 8);
    L.h = take(size_t(Tc) * (K + 1) * ff * 4);
    L.hq = take(size_t(Tc) * (K + 1) * ff);
    L.ha = take(size_t(Tc) * (K + 1) * (ff / kQ8) * 4);
    L.hc = take(size_t(Tc) * (K + 1) * (ff / kQ8) * 4);
    L.y = take(size_t(Tc) * K * n * 4);
    L.ysh = take(size_t(Tc) * n * 4);
    L.total = off;
    return L;
}

// ---------------------------------------------------------------------------------------------
// Q8 quantization of 32 values held one per lane: returns the code; lane 0 gets scale and sum.
// quant/q2_0/q2_0.cpp:101-113: d = amax / 127, id = 1 / d, q = roundf(v * id), d through fp16.
// `partner`: with activation blocks of 64 (moe_q2::run's block64 option, kernels/cuda/moe_q2.cu:58-77)
// the value at the same place of the other half of the 64-block, which shares the scale; else 0.
__device__ __forceinline__ int q8_block(float v, float& d_out, int& sum_out, float partner = 0.0f) {
    float am = fmaxf(fabsf(v), fabsf(partner));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
    const float d = __fdiv_rn(am, 127.0f);
    const float id = d != 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
    const int q = int(round_half_away(__fmul_rn(v, id)));
    int s = q;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    d_out = __half2float(__float2half_rn(d));
    sum_out = s;
    return q;
}

// x [T][n] -> q [T][n], d [T][n/32], and (optionally) the block sums of the codes.
__global__ void __launch_bounds__(256) k_quant_q8(const float* __restrict__ x, size_t n_blocks, int8_t* __restrict__ q,
                                                  float* __restrict__ d, int32_t* __restrict__ sums) {
    const size_t blk = size_t(blockIdx.x) * 8 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (blk >= n_blocks) return;
    float dd;
    int ss;
    const int c = q8_block(x[blk * kQ8 + lane], dd, ss);
    q[blk * kQ8 + lane] = int8_t(c);
    if (lane == 0) {
        d[blk] = dd;
        if (sums) sums[blk] = ss;
    }
}

// The same with a thread owning four consecutive values (x 16-byte aligned, q 4-byte aligned): one
// 16-byte load and one word of codes per thread, eight neighbouring lanes one block.
__global__ void __launch_bounds__(256) k_quant_q8_quads(const float* __restrict__ x, size_t n_blocks, int8_t* __restrict__ q,
                                                        float* __restrict__ d) {
    const size_t quad = size_t(blockIdx.x) * 256 + threadIdx.x;
    const bool live = quad < n_blocks * 8;   // no early exit: the shuffles need the whole warp
    const float4 v = live ? reinterpret_cast<const float4*>(x)[quad] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    const float hv[4] = {v.x, v.y, v.z, v.w};
    float am = fmaxf(fmaxf(fabsf(hv[0]), fabsf(hv[1])), fmaxf(fabsf(hv[2]), fabsf(hv[3])));
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
    const float dd = __fdiv_rn(am, 127.0f);
    const float id = dd != 0.0f ? __fdiv_rn(1.0f, dd) : 0.0f;
    uint32_t word = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) word |= uint32_t(int(round_half_away(__fmul_rn(hv[i], id))) & 0xff) << (8 * i);
    if (!live) return;
    reinterpret_cast<uint32_t*>(q)[quad] = word;
    if ((quad & 7) == 0) d[quad >> 3] = __half2float(__float2half_rn(dd));
}

// Activations in the form the expert kernel consumes, one row per token (x) or per slot (h):
//   q [row][k]     int8 codes in MMA-B fragment order: the four bytes of element group
//                  (b, s, hi, t) -- elements 64b + 32s + 16hi + 4t .. +3 -- are word
//                  (b * 4 + t) * 4 + s * 2 + hi, so lane (g, t) of a warp finds the B fragments of
//                  block b for its token in one 16-byte load;
//   a [row][k/32]  the block scale d (through fp16), divided by 16 for the second half of a
//                  64-block (see group_mma);
//   c [row][k/32]  the int32 kMagicBits - sum(codes) (the sum times 16 for the second half), stored
//                  through a float pointer: the value an MMA accumulator starts from, so that it
//                  ends as kMagicBits + sum((q - 1) * code), which read as a float is kMagic plus
//                  that sum, exactly.
// A thread owns four consecutive values (one 16-byte load, one word of codes out), eight
// neighbouring lanes one 32-block: `quad` is the index of the thread's four values, all lanes of a
// warp call it together, `live` is false beyond the end. With `block64` the scale is shared by the
// two 32-blocks of a 64-block (moe_q2::run's block64 option, kernels/cuda/moe_q2.cu:58-77).
__device__ __forceinline__ void quant_frag_quad(const float* __restrict__ x, int k, size_t quad, bool live, int8_t* __restrict__ q,
                                                float* __restrict__ a, float* __restrict__ c, bool block64 = false) {
    const float4 v = live ? reinterpret_cast<const float4*>(x)[quad] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    const float hv[4] = {v.x, v.y, v.z, v.w};
    float am = fmaxf(fmaxf(fabsf(hv[0]), fabsf(hv[1])), fmaxf(fabsf(hv[2]), fabsf(hv[3])));
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
    if (block64) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 8));   // sixteen lanes hold one 64-block
    const float d = __fdiv_rn(am, 127.0f);
    const float id = d != 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
    int code[4], sum = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        code[i] = int(round_half_away(__fmul_rn(hv[i], id)));
        sum += code[i];
    }
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (!live) return;
    const size_t blk = quad >> 3;
    const int bpr = k / kQ8, j = int(quad & 7);
    const size_t row = blk / bpr;
    const int rb = int(blk % bpr), b = rb >> 1, s = rb & 1, hi = j >> 2, t = j & 3;
    reinterpret_cast<uint32_t*>(q + row * k)[(b * 4 + t) * 4 + s * 2 + hi] =
        uint32_t(code[0] & 0xff) | (uint32_t(code[1] & 0xff) << 8) | (uint32_t(code[2] & 0xff) << 16) | (uint32_t(code[3] & 0xff) << 24);
    if (j == 0) {
        const float ds = __half2float(__float2half_rn(d));
        a[blk] = s ? ds * 0.0625f : ds;
        c[blk] = __int_as_float(kMagicBits - (s ? 16 * sum : sum));
    }
}
// The hidden rows: gu holds (gate x, up x) pairs; h = silu(gate x) * up x is formed here, where
// there are thousands of independent threads to hide the latency of the exponential, stored, and
// quantized like x. A thread owns four consecutive values (one word of codes in fragment order),
// eight neighbouring lanes one 32-block.
// With `slot_ids` (expert parallel), routed rows whose expert lies outside [e_lo, e_hi) are skipped:
// another rank computes them, and nothing here reads their hidden values.
__global__ void __launch_bounds__(256) k_quant_hidden(const float2* __restrict__ gu, int k, size_t n_blocks, float* __restrict__ h,
                                                      int8_t* __restrict__ q, float* __restrict__ a, float* __restrict__ c,
                                                      const int32_t* __restrict__ slot_ids, int routed_rows, int e_lo, int e_hi,
                                                      int block64, const int32_t* __restrict__ e_map,
                                                      const int32_t* __restrict__ row_list, const int* __restrict__ row_count, int store_h) {
    pdl_wait();
    pdl_trigger();
    size_t quad = size_t(blockIdx.x) * 256 + threadIdx.x;   // four values each
    size_t blk = quad >> 3;
    bool live = blk < n_blocks;   // no early exit: the shuffles below need the whole warp
    if (row_list) {
        // only the listed rows (the slots a grouping placed, in grouped order) are visited: the i-th
        // row of blocks belongs to row row_list[i]; beyond row_count there is nothing to do
        const size_t bpr = size_t(k / kQ8), i = blk / bpr;
        live = live && i < size_t(*row_count);
        if (live) {
            blk = size_t(row_list[i]) * bpr + blk % bpr;
            quad = blk * 8 + (quad & 7);
        }
    } else if (live && slot_ids) {
        const size_t r = blk / size_t(k / kQ8);
        if (r < size_t(routed_rows)) {
            const int e = slot_ids[r];
            live = e_map ? e_map[e] >= 0 : (e >= e_lo && e < e_hi);   // (ids were range-checked by the grouping kernels)
        }
    }
    const int j = int(quad & 7);        // values 4 j .. 4 j + 3 of the block
    float hv[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    if (live) {
        const float4* src = reinterpret_cast<const float4*>(gu + quad * 4);
        const float4 g0 = src[0], g1 = src[1];
        hv[0] = swiglu_ref(g0.x, g0.y);
        hv[1] = swiglu_ref(g0.z, g0.w);
        hv[2] = swiglu_ref(g1.x, g1.y);
        hv[3] = swiglu_ref(g1.z, g1.w);
        if (store_h) *reinterpret_cast<float4*>(h + quad * 4) = make_float4(hv[0], hv[1], hv[2], hv[3]);
    }
    // quant/q2_0/q2_0.cpp:101-113: d = amax / 127, id = 1 / d, q = roundf(v * id), d through fp16
    float am = fmaxf(fmaxf(fabsf(hv[0]), fabsf(hv[1])), fmaxf(fabsf(hv[2]), fabsf(hv[3])));
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
    if (block64) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 8));   // sixteen lanes hold one 64-block
    const float d = __fdiv_rn(am, 127.0f);
    const float id = d != 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
    int code[4], sum = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        code[i] = int(round_half_away(__fmul_rn(hv[i], id)));
        sum += code[i];
    }
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (!live) return;
    const int bpr = k / kQ8;
    const size_t row = blk / bpr;
    const int rb = int(blk % bpr), b = rb >> 1, s = rb & 1, hi = j >> 2, t = j & 3;
    const uint32_t word = uint32_t(code[0] & 0xff) | (uint32_t(code[1] & 0xff) << 8) | (uint32_t(code[2] & 0xff) << 16) | (uint32_t(code[3] & 0xff) << 24);
    *reinterpret_cast<uint32_t*>(q + row * k + ((b * 4 + t) * 4 + s * 2 + hi) * 4) = word;
    if (j == 0) {
        const float ds = __half2float(__float2half_rn(d));
        a[blk] = s ? ds * 0.0625f : ds;
        c[blk] = __int_as_float(kMagicBits - (s ? 16 * sum : sum));
    }
}
// Activations that arrive already quantized (natural order: codes [rows][k] int8, block scales
// [rows][k/32] float, as frx_quantize_q8 writes them) into the fragment form above: a permutation
// of the code words, the scale table, and the accumulator inputs from the block sums of the codes.
// A thread owns four consecutive codes (one word in, one word out), eight neighbouring lanes one
// 32-block.
__global__ void __launch_bounds__(256) k_q8_to_frag(const int8_t* __restrict__ xq, const float* __restrict__ xd, int k, size_t n_blocks,
                                                    int8_t* __restrict__ q, float* __restrict__ a, float* __restrict__ c) {
    const size_t quad = size_t(blockIdx.x) * 256 + threadIdx.x;
    const size_t blk = quad >> 3;
    const bool live = blk < n_blocks;   // no early exit: the shuffles below need the whole warp
    const uint32_t w = live ? reinterpret_cast<const uint32_t*>(xq)[quad] : 0u;
    int sum = __dp4a(int(w), 0x01010101, 0);   // the four signed codes added up
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (!live) return;
    const int bpr = k / kQ8, j = int(quad & 7);
    const size_t row = blk / bpr;
    const int rb = int(blk % bpr), b = rb >> 1, sh = rb & 1, hi = j >> 2, t = j & 3;
    reinterpret_cast<uint32_t*>(q + row * k)[(b * 4 + t) * 4 + sh * 2 + hi] = w;
    if (j == 0) {
        const float d = xd[blk];
        a[blk] = sh ? d * 0.0625f : d;
        c[blk] = __int_as_float(kMagicBits - (sh ? 16 * sum : sum));
    }
}

__global__ void __launch_bounds__(256) k_quant_frag(const float* __restrict__ x, int k, size_t n_blocks, int8_t* __restrict__ q,
                                                    float* __restrict__ a, float* __restrict__ c, int block64) {
    pdl_wait();
    pdl_trigger();
    const size_t quad = size_t(blockIdx.x) * 256 + threadIdx.x;   // (the number of blocks is a multiple of four: warps are live as a whole)
    quant_frag_quad(x, k, quad, quad < n_blocks * 8, q, a, c, block64 != 0);
}

// ---------------------------------------------------------------------------------------------
// Grouping: the distinct experts of up to 64 tokens in ascending id, each with its tokens in
// token order, cut into items of at most 8 tokens; then the shared expert's items; and per token
// the order in which its slots are summed (ascending expert id, the order in which the
// reference's CPU path adds them, quant/q2_0/moe_cpu.cpp:70-79). One block of 1024 threads, no
// atomics on data: the result does not depend on thread timing.
// dyn: dynamic shared memory of E * 8 + T * K * 4 bytes.
// tpi: tokens per item, 8 (the width of the MMA) or 4: with four every item takes the narrow form
// of the inner product, so all items cost the same and the even split of tasks over the SMs is an
// even split of time (an expert with more tokens is then read once from HBM and again from the L2).
// `split` (decode): how the down kernel's tasks are shared out among its blocks. A down task of an
// item of three or four tokens costs more than one of an item of one or two (two passes of float
// work per block of K instead of one), so an even split of tasks is not an even split of time:
// block b takes the tasks [ranges[b], ranges[b + 1]) (numbered item * tasks_per_expert + task),
// boundaries placed so that every block gets the same weight, a task of a small item weighing 16
// and one of a larger item `heavy`. dyn then has max_items more ints.
struct DownSplit {
    int* ranges;            // [blocks + 1], or null: no split is written
    int blocks;             // blocks of the down kernel
    int tasks_per_expert;
    int heavy;              // weight of a task of an item of more than two tokens (16 = as light ones)
    int per_item;           // weight of building an item's buffer, paid by every block that has tasks of the item
};
__device__ __forceinline__ void group_block(unsigned long long* dyn, const int32_t* __restrict__ ids, int T, int K, int E, int e_lo,
                                            int e_hi, const uint8_t* __restrict__ experts, size_t stride,
                                            const uint8_t* __restrict__ shared, Item* __restrict__ items, int* __restrict__ status,
                                            int32_t* __restrict__ order, int max_items, int tpi, bool zero_counters = false,
                                            DownSplit split = DownSplit{nullptr, 0, 0, 16, 0}, int sh_lo = 0, int sh_hi = 1 << 30) {
    // the shared expert is applied to tokens [sh_lo, sh_hi) (all of them unless the caller deals them among ranks)
    sh_lo = max(sh_lo, 0);
    sh_hi = max(min(sh_hi, T), sh_lo);
    unsigned long long* mask = dyn;   // [E] tokens routed to each expert, then the ids [T * K], the items' weights (with `split`: max_items), [E] ints
    __shared__ int warp_tot[32];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    int32_t* sid = reinterpret_cast<int32_t*>(mask + E);   // the ids, read many times below
    int* wgt = sid + T * K;                                // with `split`: weight of a task of every item, then their running sums
    if (tid == 0 && status[3] != kCookie) {   // first use of this workspace
        status[0] = kDevOk;
        status[2] = 0;
        status[3] = kCookie;
    }
    for (int e = tid; e < E; e += 1024) mask[e] = 0ull;
    __syncthreads();
    for (int s = tid; s < T * K; s += 1024) {
        const int e = ids[s];
        sid[s] = e;
        if (e < 0 || e >= E) {
            status[0] = kDevBadExpertId;
            status[2] = s;
        } else if (e >= e_lo && e < e_hi) {   // expert parallel: only the experts held here
            atomicOr(&mask[e], 1ull << (s / K));
        }
    }
    __syncthreads();
    const int per = (E + 1023) / 1024, e0 = tid * per, e1 = min(E, e0 + per);
    // one scan for two sums: the items in the low 12 bits, the weights of their tasks above (see DownSplit)
    constexpr int kCntBits = 12, kCntMask = (1 << kCntBits) - 1;
    auto weight_of = [&](int m) { return m <= 2 ? 16 : split.heavy; };
    int cnt = 0;
    for (int e = e0; e < e1; ++e) {
        const int pc = __popcll(mask[e]), full = pc / tpi, rem = pc - full * tpi;
        cnt += full + (rem ? 1 : 0);
        if (split.ranges) cnt += (full * weight_of(tpi) + (rem ? weight_of(rem) : 0)) << kCntBits;
    }
    int inc = cnt;   // inclusive scan over the block: within the warp, then over the warp totals
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += v;
    }
    if (lane == 31) warp_tot[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        int w = warp_tot[lane];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int v = __shfl_up_sync(0xffffffffu, w, o);
            if (lane >= o) w += v;
        }
        warp_tot[lane] = w;
    }
    __syncthreads();
    const int before = inc - cnt + (warp ? warp_tot[warp - 1] : 0);
    int at = before & kCntMask, wat = before >> kCntBits;   // this thread's first item, and the weight in front of it
    const int routed_items = warp_tot[31] & kCntMask, routed_weight = warp_tot[31] >> kCntBits;
    const int shared_items = shared ? (sh_hi - sh_lo + tpi - 1) / tpi : 0;
    if (routed_items + shared_items > max_items) {
        if (tid == 0) {
            status[0] = kDevTooManyItems;
            status[1] = 0;
        }
        return;
    }
    // every expert's first item and the weight in front of it, for the pass over the slots below
    int* ebase = wgt + (split.ranges ? max_items : 0);   // [E]: item index in the low 12 bits, weight above
    // the items are put together in shared memory and copied out in whole 16-byte vectors: scattered
    // 4-byte stores to global memory from this one block cost several microseconds
    Item* items_s = reinterpret_cast<Item*>(reinterpret_cast<uintptr_t>(ebase + E + 3) & ~uintptr_t(15));
    for (int e = e0; e < e1; ++e) {
        const int pc = __popcll(mask[e]), full = pc / tpi, rem = pc - full * tpi;
        ebase[e] = at | (wat << kCntBits);
        at += full + (rem ? 1 : 0);
        wat += full * weight_of(tpi) + (rem ? weight_of(rem) : 0);
    }
    __syncthreads();
    // One thread per slot: the slot's place among its expert's tokens (token order) gives its item
    // and its position there; the thread of an item's first slot also writes the item's header. Of
    // several slots of one token that name the same expert only the first is computed.
    for (int s = tid; s < T * K; s += 1024) {
        const int e = sid[s], t = s / K, k = s - t * K;
        if (e < e_lo || e >= e_hi || e < 0 || e >= E) continue;
        bool first = true;
        for (int j = 0; j < k; ++j) first = first && sid[t * K + j] != e;
        if (!first) continue;
        const unsigned long long mk = mask[e];
        const int idx = __popcll(mk & ((1ull << t) - 1ull)), pc = __popcll(mk);
        const int j = idx / tpi, pos = idx - j * tpi, eb = ebase[e];
        Item* it = items_s + (eb & kCntMask) + j;
        it->slot[pos] = s;
        if (pos == 0) {
            const int m = min(tpi, pc - j * tpi);
            it->blob = experts + size_t(e - e_lo) * stride;
            it->n_tok = m;
            it->expert = e;
            for (int z = m; z < kTokPerItem; ++z) it->slot[z] = 0;
            if (split.ranges) wgt[(eb & kCntMask) + j] = (eb >> kCntBits) + j * weight_of(tpi);   // the expert's items in front are full
        }
    }
    if (tid < shared_items) {
        Item it;
        it.blob = shared;
        it.expert = -1;
        const int t0 = sh_lo + tid * tpi, m = min(tpi, sh_hi - t0);
        it.n_tok = m;
        for (int j = 0; j < kTokPerItem; ++j) it.slot[j] = j < m ? T * K + t0 + j : 0;
        if (split.ranges) wgt[routed_items + tid] = routed_weight + tid * weight_of(tpi);   // (all but the last shared item are full)
        items_s[routed_items + tid] = it;
    }
    __syncthreads();
    for (int i = tid; i < (routed_items + shared_items) * int(sizeof(Item) / 16); i += 1024)
        reinterpret_cast<uint4*>(items)[i] = reinterpret_cast<const uint4*>(items_s)[i];
    if (tid == 0) status[1] = routed_items + shared_items;
    if (zero_counters)
        for (int i = tid; i < routed_items + shared_items; i += 1024) status[kStatusWords + i] = 0;
    // Slots of a token by ascending expert id: slot s takes the place given by the number of the
    // token's slots that come before it (smaller id, or the same id and a smaller k).
    for (int s = tid; s < T * K; s += 1024) {
        const int t = s / K, k = s - t * K, e = sid[s];
        int rank = 0;
        for (int j = 0; j < K; ++j) {
            const int ej = sid[t * K + j];
            rank += (ej < e || (ej == e && j < k)) ? 1 : 0;
        }
        order[t * K + rank] = (e < e_lo || e >= e_hi) ? -1 - s : s;   // slots of experts held elsewhere take no part in this rank's sum
    }
    if (!split.ranges) return;
    // every boundary by bisection over the running weights
    const int n_items = routed_items + shared_items;
    __syncthreads();
    if (tid <= split.blocks && n_items > 0) {
        const int tpe = split.tasks_per_expert;
        const int last_w = shared_items ? weight_of(min(tpi, sh_hi - sh_lo - (shared_items - 1) * tpi)) : 0;
        const unsigned total_w = unsigned(shared_items ? wgt[n_items - 1] + last_w : routed_weight);
        // an item also costs every block that touches it one item buffer: `per_item`, in the same units, in front of its tasks
        const unsigned per_item = unsigned(split.per_item);
        auto begins = [&](int i) { return unsigned(wgt[i]) * unsigned(tpe) + unsigned(i) * per_item; };   // weight in front of item i
        if (tid == split.blocks) {
            split.ranges[tid] = n_items * tpe;
        } else {
            const unsigned all = total_w * unsigned(tpe) + unsigned(n_items) * per_item;
            const unsigned target = unsigned((unsigned long long)all * unsigned(tid) / unsigned(split.blocks));
            int lo = 0, hi = n_items - 1;   // the last item that begins at or before the target
            while (lo < hi) {
                const int mid = (lo + hi + 1) >> 1;
                if (begins(mid) <= target) lo = mid;
                else hi = mid - 1;
            }
            const unsigned wi = (lo + 1 < n_items ? unsigned(wgt[lo + 1]) : total_w) - unsigned(wgt[lo]);   // weight of one task of the item
            const unsigned into = target - begins(lo);
            const int task = into <= per_item ? 0 : int((into - per_item) / wi);
            split.ranges[tid] = lo * tpe + min(task, tpe - 1);
        }
    }
}

// The head of a decode step, one launch of clusters of kHeadCluster blocks. Cluster 0 routes the
// tokens (when given the router's logits; token t by warp t / kHeadCluster of block
// t % kHeadCluster), meets at the cluster's hardware barrier, and its block 0 groups the tokens
// into work items. All other blocks quantize x into the expert kernel's activation form; the two
// halves do not depend on each other.
constexpr int kHeadCluster = 8;
template <int V>   // router: logits per lane, E <= 32 * V; 0: no router
__global__ void __launch_bounds__(1024) k_prologue(const float* __restrict__ logits, int32_t* __restrict__ ids, float* __restrict__ wts,
                                                   int T, int K, int E, int e_lo, int e_hi, const uint8_t* __restrict__ experts,
                                                   size_t stride, const uint8_t* __restrict__ shared, Item* __restrict__ items,
                                                   int* __restrict__ status, int32_t* __restrict__ order, int max_items,
                                                   const float* __restrict__ x, int n, size_t n_blocks, int8_t* __restrict__ xq,
                                                   float* __restrict__ xa, float* __restrict__ xc, int tpi, DownSplit split, int sh_lo, int sh_hi,
                                                   unsigned long long* stamps) {   // measurement aid (else null): four globaltimer values of block 0
    extern __shared__ unsigned long long dyn[];
    if (threadIdx.x == 0) {   // while the kernels in front still run: the translations of what this block will touch
        if (blockIdx.x < kHeadCluster) {
            const int t = blockIdx.x < T ? blockIdx.x : 0;
            if (logits) touch_l2(logits + size_t(t) * E);
            touch_l2(ids + size_t(t) * K);
            touch_l2(wts + size_t(t) * K);
            if (blockIdx.x == 0) {
                touch_l2(items);
                touch_l2(status);
                touch_l2(order);
                if (split.ranges) touch_l2(split.ranges);
            }
        } else {
            touch_l2(x);
            touch_l2(xq);
            touch_l2(xa);
            touch_l2(xc);
        }
    }
    pdl_wait();
    pdl_trigger();
    if (stamps && blockIdx.x == 0 && threadIdx.x == 0) stamps[0] = global_ns();   // the kernels in front have ended
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (blockIdx.x >= kHeadCluster) {
        const size_t qb = blockIdx.x - kHeadCluster, nqb = gridDim.x - kHeadCluster;
        for (size_t quad = qb * 1024 + threadIdx.x; quad < n_blocks * 8; quad += nqb * 1024) quant_frag_quad(x, n, quad, true, xq, xa, xc);
        return;
    }
    const int rank = int(cluster_ctarank());   // cluster 0 is blocks 0 .. kHeadCluster - 1
    if constexpr (V > 0) {
        for (int t = warp * kHeadCluster + rank; t < T; t += 32 * kHeadCluster)
            route_warp<V>(logits + size_t(t) * E, E, K, lane, ids + size_t(t) * K, wts + size_t(t) * K, nullptr, nullptr);
    }
    if (stamps && blockIdx.x == 0 && threadIdx.x == 0) stamps[1] = global_ns();   // block 0's tokens are routed
    cluster_sync_all();   // every block's ids are visible to block 0
    if (stamps && blockIdx.x == 0 && threadIdx.x == 0) stamps[2] = global_ns();   // all tokens are routed
    if (rank == 0) group_block(dyn, ids, T, K, E, e_lo, e_hi, experts, stride, shared, items, status, order, max_items, tpi, true, split, sh_lo, sh_hi);
    if (stamps && blockIdx.x == 0) {
        __syncthreads();
        if (threadIdx.x == 0) stamps[3] = global_ns();   // the work items are written
    }
}

// ---------------------------------------------------------------------------------------------
// The streaming expert kernel, used for both halves of the FFN.
//   GATE_UP: a task is two gate/up groups (each 8 gate + 8 up rows over K = n); the activations are the
//            Q8 form of x; the epilogue is SwiGLU and a float store of the hidden value.
//   else   : a task is kDownGroups down groups (16 rows each over K = ff); the activations are
//            the Q8 form of the hidden rows; the epilogue stores the expert's output rows.
// A task is one contiguous byte range of an expert blob, fetched as `cpt` chunks into ring slots:
// a down chunk is a run of whole groups (one TMA bulk copy); a gate/up chunk is the same K range
// of the task's two groups (two bulk copies on one barrier). A warp walks K once for a pair of
// groups, so the activation fragments, scales and biases of a block are read once per 32 rows.
// Task i of a block belongs to warp i % NW. Every warp owns `rpw` ring slots and is its own
// producer: it issues the copy of a later chunk into a slot as soon as it has finished with the
// chunk that was there, so slots are filled and drained strictly in order (a warp never waits on
// an mbarrier phase before it has consumed the one before) and no "empty" barriers are needed.
// While a warp computes on one chunk, its next rpw - 1 chunks are in flight.
constexpr int kDownGroups = 4;

struct StreamParams {
    const Item* items;
    int* status;
    // activations in k_quant_frag's form: of x (rows = tokens) for GATE_UP, of h (rows = slots) for down
    const int8_t* aq;
    const float* aa;
    const float* ac;
    const int32_t* slot_ids;   // expert parallel: the expert of every routed slot (else null), and the range held here
    int e_lo, e_hi;
    const int32_t* row_list;   // the hidden-row quantizer visits only these rows, *row_count of them (prefill: the grouped slots)
    const int* row_count;
    const int32_t* e_map;      // or, instead of a range: for every expert its index among those held here, -1 if elsewhere
    float2* gu;        // [slots][ff]   (gate x, up x) per hidden element, written by GATE_UP
    float* h;          // [slots][ff]   the hidden values silu(gate x) * up x, written by the quantizer of the hidden rows
    float* y;          // [T*K][n]      routed slots (down)
    float* ysh;        // [T][n]        shared-expert slots (down)
    int n, ff, K, TK;
    int cpt;           // chunks per task
    int rpw;           // ring slots per consumer warp
    int nbuf;          // item buffers (2 or 3)
    unsigned long long wait_ns;   // the longest a wait on a shared-memory barrier may last
    int block64;       // hidden rows quantized with one scale per 64 values (moe_q2::run's block64 option)
    int y_bf16;        // down: y holds bf16 rows (moe_q2::run's yd_bf16 option)
    int narrow;        // items of at most kNarrowTok tokens take units_mma_narrow (results are the same bits either way)
    unsigned long long* stamps;   // measurement aid (else null): per block four globaltimer values, see frx_debug_set_stream_stamps
    const int* ranges; // down: block b takes the tasks [ranges[b], ranges[b + 1]) (else null: an even split)
    int stream_once;   // the expert weights are read once per launch (decode): their L2 lines are marked evict-first
    int from_gu;       // down: item buffers are built from gu (SwiGLU and quantization on the way), there is no separate quantizer launch
    int* cnt;          // k_ffn: per item, the gate/up tasks finished so far
    int cpt_dn;        // k_ffn: chunks per down task (cpt: per gate/up task)
    int nbuf_dn;       // k_ffn: item buffers of the down half (nbuf: of the gate/up half)
};

// Shared-memory plan of k_stream. The activation operand of an item (fragments, scales, biases,
// the item header) lives in one of `nbuf` buffers.
constexpr int kMaxItemBufs = 3;
struct SmemPlan {
    uint32_t ring, bfrag, da, ci, item, bars, abort, total;   // bfrag, da, ci, item: buffer 0; buffer b follows at b * its size
};
__host__ __device__ inline SmemPlan smem_plan(int kdim, uint32_t chunk_bytes, int slots, int nbuf) {
    const uint32_t nb = uint32_t(kdim / kQK);
    SmemPlan s{};
    uint32_t off = 0;
    s.ring = off;
    off += uint32_t(slots) * chunk_bytes;
    off = (off + 127u) & ~127u;
    s.bfrag = off;
    off += uint32_t(nbuf) * nb * 512;   // [buffer][block][lane] uint4
    s.da = off;
    off += uint32_t(nbuf) * nb * 64;    // [buffer][block][t4] float4
    s.ci = off;
    off += uint32_t(nbuf) * nb * 128;   // [buffer][block][t4][half] int4
    s.item = off;
    off += uint32_t(nbuf) * 64;
    s.bars = off;          // `slots` ring barriers, then kMaxItemBufs "ready" and kMaxItemBufs "done" barriers
    off += uint32_t(slots + 2 * kMaxItemBufs) * 8;
    off = (off + 15u) & ~15u;
    s.abort = off;
    off += 16;
    s.total = off;
    return s;
}

// `count` units of 16 M rows against the item's tokens, continuing the running sums:
// acc_lo = {M row g, column 2*t4; M row g, column 2*t4+1}, acc_hi = the same columns of M row g + 8.
// `units` points at the first unit in shared memory, `b0` is the index of its first 64-block.
//
// Per 64-weight block two MMAs, one per 32-value activation block. The 2-bit fields of a code
// word sit at bits 0, 2, 4, 6 of each byte; the first MMA takes fields 0 and 1 (w and w >> 2
// masked with 0x03), the second takes fields 2 and 3 *in place* (masked with 0x30, i.e. the
// codes times 16), so one shift serves both. The factor 16 is undone exactly by the activation
// scale table, which holds d / 16 for the second half. Every accumulator starts at the table's
// kMagicBits - sum(a) of its token column (times 16 for the second half; the four accumulator
// inputs of a lane are one 16-byte load, used as they come and left intact for the second group),
// so it ends as kMagicBits + sum((q - 1) * a): read as a float and with kMagic subtracted, exactly
// the block's integer dot product.
// Two groups of 16 M rows (group 1 at units + gstride) share the activation fragments, scales and
// biases of each block, which are read once for both.
template <int UPC>   // units per call when known at compile time, else 0
__device__ __forceinline__ void units_mma(const uint8_t* __restrict__ units, uint32_t gstride, int count, int b0,
                                          const uint4* __restrict__ bfrag, const ulonglong2* __restrict__ da,
                                          const int4* __restrict__ ci, int lane, uint64_t (&acc_lo)[2], uint64_t (&acc_hi)[2]) {
    const int g = lane >> 2, t4 = lane & 3;
    constexpr uint32_t M0 = 0x03030303u, M1 = 0x30303030u;
    const uint8_t* codes = units + lane * 16;
    const uint8_t* scales = units + kUnitCodeBytes + g * 8;
    const uint4* bf_p = bfrag + b0 * 32 + lane;
    const int4* ci_p = ci + (b0 * 4 + t4) * 2;
    const uint64_t neg_magic = pack2(-kMagic, -kMagic);
    const ulonglong2* da_p = da + b0 * 4 + t4;
    const int n_units = UPC ? UPC : count;
#pragma unroll(2)
    for (int u = 0; u < n_units; ++u) {
        uint4 c[2];
        uint2 sc[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            c[r] = *reinterpret_cast<const uint4*>(codes + r * gstride + u * kUnitBytes);
            sc[r] = *reinterpret_cast<const uint2*>(scales + r * gstride + u * kUnitBytes);
        }
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int b = 2 * u + j;
            const uint4 bf = bf_p[b * 32];
            const int4 cq0 = ci_p[b * 8], cq1 = ci_p[b * 8 + 1];   // accumulator inputs: kMagicBits - sum(codes), per column, both halves
            const ulonglong2 a = da_p[b * 4];   // {a0[c0], a0[c1]}, {a1[c0] / 16, a1[c1] / 16}
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                const uint32_t w0 = j ? c[r].y : c[r].x, w1 = j ? c[r].w : c[r].z;
                const uint32_t v0 = w0 >> 2, v1 = w1 >> 2;
                uint64_t lo0, hi0, lo1, hi1;
                mma_u8s8_c4(lo0, hi0, w0 & M0, w1 & M0, v0 & M0, v1 & M0, bf.x, bf.y, cq0);
                mma_u8s8_c4(lo1, hi1, w0 & M1, w1 & M1, v0 & M1, v1 & M1, bf.z, bf.w, cq1);
                const __half2 s_lo = *reinterpret_cast<const __half2*>(&sc[r].x), s_hi = *reinterpret_cast<const __half2*>(&sc[r].y);
                const float d_lo = j ? __high2float(s_lo) : __low2float(s_lo);
                const float d_hi = j ? __high2float(s_hi) : __low2float(s_hi);
                // a0 * S0 and (a1 / 16) * (16 * S1) are exact (11-bit scale x 13-bit integer), so one fused
                // multiply-add rounds exactly where the reference's two statements round once.
                const uint64_t sumi_lo = fma2(a.y, add2(lo1, neg_magic), mul2(a.x, add2(lo0, neg_magic)));
                const uint64_t sumi_hi = fma2(a.y, add2(hi1, neg_magic), mul2(a.x, add2(hi0, neg_magic)));
                // The weight scale is applied with scalar multiplies: a packed multiply followed by a
                // packed add is contracted into one fused multiply-add by the assembler, which would
                // round once where the reference rounds twice.
                float s0, s1, s2, s3;
                unpack2(sumi_lo, s0, s1);
                unpack2(sumi_hi, s2, s3);
                acc_lo[r] = add2(acc_lo[r], pack2(__fmul_rn(d_lo, s0), __fmul_rn(d_lo, s1)));
                acc_hi[r] = add2(acc_hi[r], pack2(__fmul_rn(d_hi, s2), __fmul_rn(d_hi, s3)));
            }
        }
    }
}

// The narrow form of units_mma, for items of at most kNarrowTok tokens (most items of a decode
// batch: with 64 tokens over 512 experts an expert gets 1.75 tokens on average). The MMA's eight
// token columns are used twice: the B operand of row group 0 carries the item's tokens in columns
// 0..3 and zeros in columns 4..7, the B operand of row group 1 zeros in columns 0..3 and the tokens
// in columns 4..7, and the two MMAs accumulate into one D. Lanes t4 = 0, 1 then hold group 0's sums
// of tokens (0, 1) and (2, 3), lanes t4 = 2, 3 those of group 1, so every lane's float work is on
// live values and there is half as much of it per row. Products, scaling and the order of the
// additions per (row, token) are those of units_mma: the results are the same bits.
// The item buffer must have been built for the narrow form (see build in k_stream): zeros in token
// columns 4..7 of the B fragments, scale and bias entries of lanes t4 = 2, 3 equal to those of t4 = 0, 1.
template <int UPC, int BS = 32>   // BS: 16-byte vectors per block of the B fragments (32: eight token columns; 16: four)
__device__ __forceinline__ void units_mma_narrow(const uint8_t* __restrict__ units, uint32_t gstride, int count, int b0,
                                                 const uint4* __restrict__ bfrag, const ulonglong2* __restrict__ da,
                                                 const int4* __restrict__ ci, int lane, uint64_t& acc_lo, uint64_t& acc_hi) {
    const int g = lane >> 2, t4 = lane & 3;
    constexpr uint32_t M0 = 0x03030303u, M1 = 0x30303030u;
    const uint8_t* codes = units + lane * 16;
    const uint8_t* scales = units + (t4 >> 1) * gstride + kUnitCodeBytes + g * 8;   // of the lane's own row group
    // B operand: lanes g < 4 carry token g for row group 0 and zeros for row group 1, lanes g >= 4
    // zeros for group 0 and token g - 4 for group 1. The zeros never change, so each lane loads only
    // its live fragment (a predicated load: half the shared-memory traffic of two full loads).
    const uint32_t bf_a = smem_u32(bfrag + b0 * BS + (g & 3) * 4 + t4);
    const bool low = g < 4;
    uint4 bfa = make_uint4(0u, 0u, 0u, 0u), bfb = bfa;
    const ulonglong2* nm_p = reinterpret_cast<const ulonglong2*>(ci + (b0 * 4 + t4) * 2);   // -(kMagic + sum of the codes), see build
    const ulonglong2* da_p = da + b0 * 4 + t4;
    const int n_units = UPC ? UPC : count;
#pragma unroll(2)
    for (int u = 0; u < n_units; ++u) {
        const uint4 c0 = *reinterpret_cast<const uint4*>(codes + u * kUnitBytes);
        const uint4 c1 = *reinterpret_cast<const uint4*>(codes + gstride + u * kUnitBytes);
        const uint2 sc = *reinterpret_cast<const uint2*>(scales + u * kUnitBytes);
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int b = 2 * u + j;
            lds128_if(bfa, bf_a + b * (BS * 16), low);
            lds128_if(bfb, bf_a + b * (BS * 16), !low);
            const ulonglong2 nm = nm_p[b * 8];   // {first half: columns c0, c1}, {second half}
            const ulonglong2 a = da_p[b * 4];
            const uint32_t w0 = j ? c0.y : c0.x, w1 = j ? c0.w : c0.z;   // group 0: rows g, g + 8
            const uint32_t x0 = j ? c1.y : c1.x, x1 = j ? c1.w : c1.z;   // group 1
            const uint32_t v0 = w0 >> 2, v1 = w1 >> 2, y0 = x0 >> 2, y1 = x1 >> 2;
            uint64_t lo0, hi0, lo1, hi1;
            mma_u8s8_chain2(lo0, hi0, w0 & M0, w1 & M0, v0 & M0, v1 & M0, bfa.x, bfa.y, x0 & M0, x1 & M0, y0 & M0, y1 & M0, bfb.x, bfb.y, kMagicBits);
            mma_u8s8_chain2(lo1, hi1, w0 & M1, w1 & M1, v0 & M1, v1 & M1, bfa.z, bfa.w, x0 & M1, x1 & M1, y0 & M1, y1 & M1, bfb.z, bfb.w, kMagicBits);
            const __half2 s_lo = *reinterpret_cast<const __half2*>(&sc.x), s_hi = *reinterpret_cast<const __half2*>(&sc.y);
            const float d_lo = j ? __high2float(s_lo) : __low2float(s_lo);
            const float d_hi = j ? __high2float(s_hi) : __low2float(s_hi);
            const uint64_t sumi_lo = fma2(a.y, add2(lo1, nm.y), mul2(a.x, add2(lo0, nm.x)));
            const uint64_t sumi_hi = fma2(a.y, add2(hi1, nm.y), mul2(a.x, add2(hi0, nm.x)));
            float s0, s1, s2, s3;   // scalar multiplies by the weight scale, as in units_mma
            unpack2(sumi_lo, s0, s1);
            unpack2(sumi_hi, s2, s3);
            acc_lo = add2(acc_lo, pack2(__fmul_rn(d_lo, s0), __fmul_rn(d_lo, s1)));
            acc_hi = add2(acc_hi, pack2(__fmul_rn(d_hi, s2), __fmul_rn(d_hi, s3)));
        }
    }
}

// Four row groups at once for items of one or two tokens: the B operand of group j carries the
// tokens in columns 2j, 2j + 1 and zeros elsewhere, the four MMAs accumulate into one D, and lane
// (g, t4) finishes group t4: a quarter of the float work of units_mma per row, all of it live.
// `units` points at the first unit of group 0 of the chunk, group j follows at j * gstride. The item
// buffer is in the narrow form (zeros in token column 4; scale and bias entries of tokens 0, 1 at
// the quad of lanes t4 = 0). Same products, same scaling, same order of additions per (row, token).
template <int UPC, int BS = 32>
__device__ __forceinline__ void units_mma_n2(const uint8_t* __restrict__ units, uint32_t gstride, int count, int b0,
                                             const uint4* __restrict__ bfrag, const ulonglong2* __restrict__ da, const int4* __restrict__ ci,
                                             int lane, uint64_t& acc_lo, uint64_t& acc_hi) {
    const int g = lane >> 2, t4 = lane & 3;
    constexpr uint32_t M0 = 0x03030303u, M1 = 0x30303030u;
    const uint8_t* codes = units + lane * 16;
    const uint8_t* scales = units + t4 * gstride + kUnitCodeBytes + g * 8;   // of the lane's own row group
    // B operand of row group j: token g & 1 in the lanes with g >> 1 == j, zeros elsewhere; a lane loads
    // only its live fragment, the zeros of the other three stay in registers
    const uint32_t bf_a = smem_u32(bfrag + b0 * BS + (g & 1) * 4 + t4);
    uint4 bf[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) bf[j] = make_uint4(0u, 0u, 0u, 0u);
    const ulonglong2* nm_p = reinterpret_cast<const ulonglong2*>(ci + b0 * 8);
    const ulonglong2* da_p = da + b0 * 4;
    const int n_units = UPC ? UPC : count;
#pragma unroll(1)
    for (int u = 0; u < n_units; ++u) {
        uint4 c[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) c[j] = *reinterpret_cast<const uint4*>(codes + j * gstride + u * kUnitBytes);
        const uint2 sc = *reinterpret_cast<const uint2*>(scales + u * kUnitBytes);
#pragma unroll
        for (int jj = 0; jj < 2; ++jj) {
            const int b = 2 * u + jj;
            const ulonglong2 nm = nm_p[b * 8];
            const ulonglong2 a = da_p[b * 4];
            uint32_t a0[16], a1[16], bb0[8], bb1[8];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                lds128_if(bf[j], bf_a + b * (BS * 16), (g >> 1) == j);
                bb0[2 * j] = bf[j].x;
                bb0[2 * j + 1] = bf[j].y;
                bb1[2 * j] = bf[j].z;
                bb1[2 * j + 1] = bf[j].w;
                const uint32_t w0 = jj ? c[j].y : c[j].x, w1 = jj ? c[j].w : c[j].z;
                const uint32_t v0 = w0 >> 2, v1 = w1 >> 2;
                a0[4 * j] = w0 & M0;
                a0[4 * j + 1] = w1 & M0;
                a0[4 * j + 2] = v0 & M0;
                a0[4 * j + 3] = v1 & M0;
                a1[4 * j] = w0 & M1;
                a1[4 * j + 1] = w1 & M1;
                a1[4 * j + 2] = v0 & M1;
                a1[4 * j + 3] = v1 & M1;
            }
            uint64_t lo0, hi0, lo1, hi1;
            mma_u8s8_chain4(lo0, hi0, a0, bb0, kMagicBits);
            mma_u8s8_chain4(lo1, hi1, a1, bb1, kMagicBits);
            const __half2 s_lo = *reinterpret_cast<const __half2*>(&sc.x), s_hi = *reinterpret_cast<const __half2*>(&sc.y);
            const float d_lo = jj ? __high2float(s_lo) : __low2float(s_lo);
            const float d_hi = jj ? __high2float(s_hi) : __low2float(s_hi);
            const uint64_t sumi_lo = fma2(a.y, add2(lo1, nm.y), mul2(a.x, add2(lo0, nm.x)));
            const uint64_t sumi_hi = fma2(a.y, add2(hi1, nm.y), mul2(a.x, add2(hi0, nm.x)));
            float s0, s1, s2, s3;   // scalar multiplies by the weight scale, as in units_mma
            unpack2(sumi_lo, s0, s1);
            unpack2(sumi_hi, s2, s3);
            acc_lo = add2(acc_lo, pack2(__fmul_rn(d_lo, s0), __fmul_rn(d_lo, s1)));
            acc_hi = add2(acc_hi, pack2(__fmul_rn(d_hi, s2), __fmul_rn(d_hi, s3)));
        }
    }
}

// Four row groups as two pairs in the narrow form (items of three or four tokens): the activation
// fragments, scales and biases of a block are loaded once and serve both pairs.
template <int UPC, int BS = 32>
__device__ __forceinline__ void units_mma_n4x2(const uint8_t* __restrict__ units, uint32_t gstride, int count, int b0,
                                               const uint4* __restrict__ bfrag, const ulonglong2* __restrict__ da, const int4* __restrict__ ci,
                                               int lane, uint64_t (&acc_lo)[2], uint64_t (&acc_hi)[2]) {
    const int g = lane >> 2, t4 = lane & 3;
    constexpr uint32_t M0 = 0x03030303u, M1 = 0x30303030u;
    const uint8_t* codes = units + lane * 16;
    const uint8_t* scales = units + (t4 >> 1) * gstride + kUnitCodeBytes + g * 8;   // pair 0; pair 1 two groups on
    const uint32_t bf_a = smem_u32(bfrag + b0 * BS + (g & 3) * 4 + t4);   // as in units_mma_narrow
    const bool low = g < 4;
    uint4 bfa = make_uint4(0u, 0u, 0u, 0u), bfb = bfa;
    const ulonglong2* nm_p = reinterpret_cast<const ulonglong2*>(ci + (b0 * 4 + t4) * 2);
    const ulonglong2* da_p = da + b0 * 4 + t4;
    const int n_units = UPC ? UPC : count;
#pragma unroll(1)
    for (int u = 0; u < n_units; ++u) {
        uint4 c[4];
        uint2 sc[2];
#pragma unroll
        for (int j = 0; j < 4; ++j) c[j] = *reinterpret_cast<const uint4*>(codes + j * gstride + u * kUnitBytes);
#pragma unroll
        for (int pi = 0; pi < 2; ++pi) sc[pi] = *reinterpret_cast<const uint2*>(scales + 2 * pi * gstride + u * kUnitBytes);
#pragma unroll
        for (int jj = 0; jj < 2; ++jj) {
            const int b = 2 * u + jj;
            lds128_if(bfa, bf_a + b * (BS * 16), low);
            lds128_if(bfb, bf_a + b * (BS * 16), !low);
            const ulonglong2 nm = nm_p[b * 8];
            const ulonglong2 a = da_p[b * 4];
#pragma unroll
            for (int pi = 0; pi < 2; ++pi) {
                const uint4 c0 = c[2 * pi], c1 = c[2 * pi + 1];
                const uint32_t w0 = jj ? c0.y : c0.x, w1 = jj ? c0.w : c0.z;
                const uint32_t x0 = jj ? c1.y : c1.x, x1 = jj ? c1.w : c1.z;
                const uint32_t v0 = w0 >> 2, v1 = w1 >> 2, y0 = x0 >> 2, y1 = x1 >> 2;
                uint64_t lo0, hi0, lo1, hi1;
                mma_u8s8_chain2(lo0, hi0, w0 & M0, w1 & M0, v0 & M0, v1 & M0, bfa.x, bfa.y, x0 & M0, x1 & M0, y0 & M0, y1 & M0, bfb.x, bfb.y, kMagicBits);
                mma_u8s8_chain2(lo1, hi1, w0 & M1, w1 & M1, v0 & M1, v1 & M1, bfa.z, bfa.w, x0 & M1, x1 & M1, y0 & M1, y1 & M1, bfb.z, bfb.w, kMagicBits);
                const __half2 s_lo = *reinterpret_cast<const __half2*>(&sc[pi].x), s_hi = *reinterpret_cast<const __half2*>(&sc[pi].y);
                const float d_lo = jj ? __high2float(s_lo) : __low2float(s_lo);
                const float d_hi = jj ? __high2float(s_hi) : __low2float(s_hi);
                const uint64_t sumi_lo = fma2(a.y, add2(lo1, nm.y), mul2(a.x, add2(lo0, nm.x)));
                const uint64_t sumi_hi = fma2(a.y, add2(hi1, nm.y), mul2(a.x, add2(hi0, nm.x)));
                float s0, s1, s2, s3;
                unpack2(sumi_lo, s0, s1);
                unpack2(sumi_hi, s2, s3);
                acc_lo[pi] = add2(acc_lo[pi], pack2(__fmul_rn(d_lo, s0), __fmul_rn(d_lo, s1)));
                acc_hi[pi] = add2(acc_hi[pi], pack2(__fmul_rn(d_hi, s2), __fmul_rn(d_hi, s3)));
            }
        }
    }
}

// The narrow forms start their accumulators at kMagicBits and add -(kMagic + sum of the codes) in
// float (exact: both are integers below 2^24); `c` is the wide form's accumulator input,
// kMagicBits - sum as an int32 behind a float pointer.
__device__ __forceinline__ float narrow_bias(float c) { return -(kMagic + float(kMagicBits - __float_as_int(c))); }

// The item buffer of a down item in the narrow form (B fragments of the item's at most kNarrowTok
// tokens, BS 16-byte vectors per block; scales; -(kMagic + sum of the codes)) straight from the
// (gate x, up x) pairs of the item's slots: h = silu(gate x) * up x is formed here and quantized as
// k_quant_hidden does (quant/q2_0/q2_0.cpp:101-113: d = amax / 127, id = 1 / d, q = roundf(v * id),
// d through fp16). A thread owns four consecutive values, eight neighbouring lanes one 32-block;
// thread btid of NT (whole warps) takes part. The pairs were written by other SMs, during this
// kernel or the one before: they are read from the L2.
template <int BS>
__device__ __noinline__ void build_hidden_narrow(const float2* __restrict__ gu, int ff, const Item* __restrict__ it, uint32_t* bw,
                                                    float* daw, float* ciw, int btid, int NT) {
    const int m = min(it->n_tok, kNarrowTok);
    const int qpr = ff / 4, total = m * qpr;   // quads per row (a multiple of 32: whole warps stay together)
    constexpr int kBatch = 2;                  // loads of this many quads are in flight together
    for (int base = 0; base < total; base += kBatch * NT) {
        float4 g0[kBatch], g1[kBatch];
#pragma unroll
        for (int k = 0; k < kBatch; ++k) {
            const int idx = base + k * NT + btid;
            if (idx < total) {
                const int g = idx / qpr, rq = idx - g * qpr;
                const float4* src = reinterpret_cast<const float4*>(gu + size_t(it->slot[g]) * ff + size_t(rq) * 4);
                g0[k] = __ldcg(src);
                g1[k] = __ldcg(src + 1);
            }
        }
#pragma unroll
        for (int k = 0; k < kBatch; ++k) {
            if (base + k * NT >= total) break;   // uniform for the warp
            const int idx = base + k * NT + btid;
            const bool live = idx < total;
            const int g = live ? idx / qpr : 0, rq = live ? idx - g * qpr : 0;
            float hv[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            if (live) {
                hv[0] = swiglu_ref(g0[k].x, g0[k].y);
                hv[1] = swiglu_ref(g0[k].z, g0[k].w);
                hv[2] = swiglu_ref(g1[k].x, g1[k].y);
                hv[3] = swiglu_ref(g1[k].z, g1[k].w);
            }
            float am = fmaxf(fmaxf(fabsf(hv[0]), fabsf(hv[1])), fmaxf(fabsf(hv[2]), fabsf(hv[3])));
#pragma unroll
            for (int o = 1; o < 8; o <<= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
            const float d = __fdiv_rn(am, 127.0f);
            const float id = d != 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
            int code[4], sum = 0;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                code[i] = int(round_half_away(__fmul_rn(hv[i], id)));
                sum += code[i];
            }
#pragma unroll
            for (int o = 1; o < 8; o <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
            if (live) {
                const int rb = rq >> 3, j = rq & 7, b = rb >> 1, h = rb & 1, hi = j >> 2, t = j & 3;
                bw[(b * BS + g * 4 + t) * 4 + h * 2 + hi] =
                    uint32_t(code[0] & 0xff) | (uint32_t(code[1] & 0xff) << 8) | (uint32_t(code[2] & 0xff) << 16) | (uint32_t(code[3] & 0xff) << 24);
                if (j == 0) {
                    const float ds = __half2float(__float2half_rn(d));
                    const float av = h ? ds * 0.0625f : ds, nv = -(kMagic + float(h ? 16 * sum : sum));
                    const int dst = (b * 4 + (g >> 1)) * 4 + h * 2 + (g & 1);
                    daw[dst] = av;
                    daw[dst + 8] = av;
                    const int cq = (b * 4 + (g >> 1)) * 8 + h * 2 + (g & 1);
                    ciw[cq] = nv;
                    ciw[cq + 16] = nv;
                }
            }
        }
    }
}

// UPC: units per units_mma call when known at compile time (gate/up: units per chunk; down: units
// per group), else 0.
// TASK4 (decode, where grouping cuts items at four tokens): a task is four groups walked once over
// K, a chunk the same K range of all four (four bulk copies on one barrier); items of one or two
// tokens take units_mma_n2, items of three or four units_mma_n4x2.
template <bool GATE_UP, int NW, int UPC, bool TASK4 = false>
__global__ void __launch_bounds__(NW * 32, 1) k_stream(const StreamParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    // Gate/up follows the kernel that makes the work items, so it waits for it at once. Down follows
    // the hidden-row quantizer, which itself started only after gate/up and therefore after the
    // items were complete: down reads the items and starts streaming its weights (constant data)
    // while the quantizer is still running, and waits for it only before it touches the hidden rows.
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // (measurement aid: nothing is kept in a register for it, the pointer is a launch parameter)
    auto stamp_now = [&](int i) {
        if (p.stamps && threadIdx.x == 0) p.stamps[size_t(blockIdx.x) * 4 + i] = global_ns();
    };
    stamp_now(0);   // the block has started
    const int kdim = GATE_UP ? p.n : p.ff;
    const int nb = kdim / kQK, units = kdim / kUnitK;
    const uint32_t group_bytes = uint32_t(units) * kUnitBytes;
    const uint32_t task_bytes = TASK4 ? group_bytes * 4 : GATE_UP ? group_bytes * 2 : group_bytes * kDownGroups;
    const int cpt = p.cpt, rpw = p.rpw;
    const uint32_t chunk_bytes = task_bytes / uint32_t(cpt);
    const uint32_t half_bytes = chunk_bytes / 2;      // gate/up: one group's share of a chunk
    const uint32_t quarter_bytes = chunk_bytes / 4;   // four-group tasks: one group's share of a chunk
    const int tasks_per_expert = TASK4 ? (GATE_UP ? p.ff / 32 : p.n / 64) : GATE_UP ? p.ff / 16 : p.n / 16 / kDownGroups;
    const size_t section = GATE_UP ? 0 : size_t(p.ff / 8) * (size_t(p.n / kUnitK) * kUnitBytes);
    const int slots = NW * rpw;
    const int nbuf = p.nbuf;
    const SmemPlan sp = smem_plan(kdim, chunk_bytes, slots, nbuf);
    uint64_t* ready = reinterpret_cast<uint64_t*>(smem + sp.bars) + slots;   // ready[b]: item buffer b is built
    uint64_t* done = ready + kMaxItemBufs;                                   // done[b]: every warp has finished with it
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + sp.bars) + warp * rpw;   // this warp's barriers
    uint8_t* ring = smem + sp.ring + size_t(warp) * rpw * chunk_bytes;            // this warp's slots
    volatile int* abort = reinterpret_cast<volatile int*>(smem + sp.abort);

    if (threadIdx.x == 32) {   // the translations of what this block will touch after its wait
        touch_l2(p.items);
        touch_l2(p.status);
        touch_l2(p.aq);
        touch_l2(p.aa);
        touch_l2(p.ac);
        touch_l2(p.gu);
        if (!GATE_UP) {
            touch_l2(p.y);
            if (p.ysh) touch_l2(p.ysh);
            if (p.ranges) touch_l2(p.ranges);
        }
    }
    if (threadIdx.x == 0) {   // (before the wait: this needs nothing from the kernels in front)
        for (int s = 0; s < slots; ++s) mbar_init(reinterpret_cast<uint64_t*>(smem + sp.bars) + s, 1);
        for (int b = 0; b < kMaxItemBufs; ++b) {
            mbar_init(ready + b, NW);
            mbar_init(done + b, NW);
        }
        *abort = 0;
        mbar_fence_init();
    }
    // The next kernel may be scheduled from here on. (Gate/up says so only after its own wait: what
    // follows it, down included, then starts after the item list is complete. Letting every kernel of
    // the chain say so first thing was measured: no gain at batch 64, a loss at small batches.)
    if (GATE_UP) pdl_wait();
    pdl_trigger();
    // (down, before its wait: the item list was complete and flushed to the L2 before the kernel in
    // front of this one began, but the same addresses are rewritten every layer, so the reads
    // bypass this SM's L1, which may still hold the previous layer's lines)
    const int n_items = GATE_UP ? p.status[1] : *reinterpret_cast<const volatile int*>(p.status + 1);
    const long long total = (long long)n_items * tasks_per_expert;
    long long lo = total * blockIdx.x / gridDim.x, hi = total * (blockIdx.x + 1) / gridDim.x;
    if (!GATE_UP && p.ranges && n_items > 0) {   // a split by weight, made by the grouping kernel
        lo = *reinterpret_cast<const volatile int*>(p.ranges + blockIdx.x);
        hi = *reinterpret_cast<const volatile int*>(p.ranges + blockIdx.x + 1);
    }
    const int ntasks = int(hi - lo);
    if (ntasks <= 0) {   // uniform for the block
        if (!GATE_UP) pdl_wait();   // keeps "this grid has ended" meaning "every kernel before it has ended"
        return;
    }
    auto item_blob = [&](int item) -> const uint8_t* {
        if (GATE_UP) return p.items[item].blob;
        return *reinterpret_cast<const uint8_t* const volatile*>(&p.items[item].blob);
    };

    __syncthreads();

    // ---- this warp's stream of chunks. Task i of the block (i = warp, warp + NW, ...) is fetched as
    // cpt chunks; chunk j of the warp goes to its ring slot j % rpw. Lane 0 issues the TMA copies:
    // the first rpw chunks up front, then chunk j + rpw into the slot that chunk j just left.
    // (Handing tasks to whichever warp is free, from a shared counter, was measured and is slower.)
    const int first_item = int(lo / tasks_per_expert), last_item = int((hi - 1) / tasks_per_expert);
    int is_item = 0, is_task = 0, is_i = warp, is_c = 0, is_slot = 0;   // the next chunk to issue
    const uint8_t* is_blob = nullptr;
    if (lane == 0) {
        const long long tau = lo + warp;
        is_item = int(tau / tasks_per_expert);
        is_task = int(tau % tasks_per_expert);
        if (is_i < ntasks) is_blob = item_blob(is_item) + section;
    }
    // weights that are read once (decode) are marked evict-first in the L2: see l2_policy_evict_first
    const uint64_t l2pol = p.stream_once ? l2_policy_evict_first() : l2_policy_evict_normal();
    auto copy = [&](void* dst, const void* src, uint32_t bytes, uint64_t* bar) { bulk_g2s_hint(dst, src, bytes, bar, l2pol); };
    auto issue_next = [&]() {   // lane 0 only
        if (is_i >= ntasks) return;
        mbar_expect_tx(full + is_slot, chunk_bytes);
        uint8_t* dst = ring + size_t(is_slot) * chunk_bytes;
        if (TASK4) {     // the same K range of the task's four groups
            const uint8_t* src = is_blob + size_t(is_task) * task_bytes + size_t(is_c) * quarter_bytes;
#pragma unroll
            for (int gq = 0; gq < 4; ++gq) copy(dst + gq * quarter_bytes, src + size_t(gq) * group_bytes, quarter_bytes, full + is_slot);
        } else if (GATE_UP) {   // the same K range of the task's two groups, one after the other
            const uint8_t* src = is_blob + size_t(is_task) * task_bytes + size_t(is_c) * half_bytes;
            copy(dst, src, half_bytes, full + is_slot);
            copy(dst + half_bytes, src + group_bytes, half_bytes, full + is_slot);
        } else {
            copy(dst, is_blob + size_t(is_task) * task_bytes + size_t(is_c) * chunk_bytes, chunk_bytes, full + is_slot);
        }
        if (++is_slot == rpw) is_slot = 0;
        if (++is_c == cpt) {
            is_c = 0;
            is_i += NW;
            is_task += NW;
            if (is_i < ntasks && is_task >= tasks_per_expert) {
                while (is_task >= tasks_per_expert) {
                    is_task -= tasks_per_expert;
                    ++is_item;
                }
                is_blob = item_blob(is_item) + section;
            }
        }
    };
    if (lane == 0)
        for (int k = 0; k < rpw; ++k) issue_next();
    int cs_slot = 0;
    uint32_t cs_phase = 0;   // the chunk being consumed: its slot and that slot's barrier phase
    auto chunk_wait = [&]() -> const uint8_t* {
        mbar_wait_bounded(full + cs_slot, cs_phase, abort, p.wait_ns);
        return ring + size_t(cs_slot) * chunk_bytes;
    };
    auto chunk_done = [&]() {
        __syncwarp();
        if (lane == 0) issue_next();   // refills the slot this chunk just left
        if (++cs_slot == rpw) {
            cs_slot = 0;
            cs_phase ^= 1u;
        }
    };

    // ---- segments of consecutive tasks that belong to one item
    const int nseg = last_item - first_item + 1;
    const int ctid = threadIdx.x;

    // btid / bthreads: this thread's index among the threads that share the build, and their number
    // (the whole block in the steady state; half of it each for the first two items, which are
    // built side by side so that their global-memory round trips overlap)
    auto build = [&](int q, int btid, int bthreads) {
        const Item* it = p.items + first_item + q;
        const int buf = q % nbuf;
        uint32_t* bw = reinterpret_cast<uint32_t*>(smem + sp.bfrag + buf * (nb * 512));
        float* daw = reinterpret_cast<float*>(smem + sp.da + buf * (nb * 64));
        float* ciw = reinterpret_cast<float*>(smem + sp.ci + buf * (nb * 128));
        if (btid < kItemWords) reinterpret_cast<uint32_t*>(smem + sp.item + buf * 64)[btid] = reinterpret_cast<const uint32_t*>(it)[btid];
        const int m = it->n_tok;
        const bool narrow = m <= kNarrowTok && p.narrow;   // see units_mma_narrow
        const int NT = bthreads;
        if (!GATE_UP && p.from_gu) {   // the hidden rows are made here (every item is narrow then)
            build_hidden_narrow<32>(p.gu, p.ff, it, bw, daw, ciw, btid, NT);
            return;
        }
        // column g of the B fragments, scales and biases <- activation row of the item's g-th slot
        const int vpr = nb * 4;   // 16-byte vectors per row
        for (int base = btid; base < m * vpr; base += 4 * NT) {
            uint4 v[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int idx = base + k * NT;
                if (idx < m * vpr) {
                    const int g = idx / vpr, r = idx % vpr;
                    const int slot = it->slot[g];
                    const size_t row = GATE_UP ? size_t(slot_token(slot, p.K, p.TK)) : size_t(slot);
                    v[k] = reinterpret_cast<const uint4*>(p.aq + row * kdim)[r];
                }
            }
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int idx = base + k * NT;
                if (idx < m * vpr) {
                    const int g = idx / vpr, r = idx % vpr;
                    reinterpret_cast<uint4*>(bw)[(r >> 2) * 32 + g * 4 + (r & 3)] = v[k];
                }
            }
        }
        for (int idx = btid; idx < m * nb * 2; idx += NT) {
            const int g = idx / (nb * 2), r = idx % (nb * 2), b = r >> 1, s = r & 1;
            const int slot = it->slot[g];
            const size_t row = GATE_UP ? size_t(slot_token(slot, p.K, p.TK)) : size_t(slot);
            const int dst = (b * 4 + (g >> 1)) * 4 + s * 2 + (g & 1);
            const float av = p.aa[row * (nb * 2) + r];
            daw[dst] = av;
            // the MMA's accumulator input of this block half: {c0, c1, c0, c1} for the lane's two token columns and both row halves
            const float cv = p.ac[row * (nb * 2) + r];
            if (narrow) {
                // one quad per (block, t4): -(kMagic + sum of the codes) for {c0, c1} of the first half and
                // {c0, c1} of the second (the sum times 16 there): the accumulators start at kMagicBits and
                // this is added to them as floats. Lanes t4 = 2, 3 work on the same tokens as t4 = 0, 1
                // (for the second row group).
                const float nv = narrow_bias(cv);
                const int cq = (b * 4 + (g >> 1)) * 8 + s * 2 + (g & 1);
                ciw[cq] = nv;
                ciw[cq + 16] = nv;
                daw[dst + 8] = av;
            } else {
                const int cq = ((b * 4 + (g >> 1)) * 2 + s) * 4 + (g & 1);
                ciw[cq] = cv;
                ciw[cq + 2] = cv;
            }
        }
    };

    // Items are pipelined through the buffers without block-wide barriers: a warp that has finished
    // its tasks of item q builds its share of item q + nbuf - 1 (into the buffer item q - 1 used, once
    // every warp has left that item) and goes on to item q + 1 as soon as all shares of it are in.
    // With three buffers a warp can run one item ahead of the slowest warp.
    // down: the output row of a slot (routed slots in y, float or bf16 rows; shared-expert slots in ysh,
    // always float), and the store of rows `row` and `row + 8` of it
    auto out_row = [&](int sl) -> float* {
        if (sl >= p.TK) return p.ysh + size_t(sl - p.TK) * p.n;
        return p.y_bf16 ? reinterpret_cast<float*>(reinterpret_cast<__nv_bfloat16*>(p.y) + size_t(sl) * p.n) : p.y + size_t(sl) * p.n;
    };
    auto put2 = [&](float* o, int row, float v0, float v8) {
        if (p.y_bf16) {
            reinterpret_cast<__nv_bfloat16*>(o)[row] = __float2bfloat16_rn(v0);
            reinterpret_cast<__nv_bfloat16*>(o)[row + 8] = __float2bfloat16_rn(v8);
        } else {
            o[row] = v0;
            o[row + 8] = v8;
        }
    };
    const int ahead = nbuf - 1;
    if (!GATE_UP) pdl_wait();   // the first weight chunks are already in flight
    stamp_now(1);   // the kernels in front have ended, the first copies are issued
    if (ahead == 2 && nseg >= 2) {   // the first two items side by side: one half of the warps each
        constexpr int H = NW / 2;
        build(warp < H ? 0 : 1, warp < H ? ctid : ctid - H * 32, warp < H ? H * 32 : (NW - H) * 32);
        __syncwarp();
        if (lane == 0) {   // every warp arrives at both barriers; they complete when the builders have
            mbar_arrive(ready + 0);
            mbar_arrive(ready + 1);
        }
    } else {
        for (int q = 0; q < ahead && q < nseg; ++q) {
            build(q, ctid, NW * 32);
            __syncwarp();
            if (lane == 0) mbar_arrive(ready + q % nbuf);
        }
    }
    for (int q = 0; q < nseg; ++q) {
        const int item = first_item + q, buf = q % nbuf;
        mbar_wait_bounded(ready + buf, uint32_t(q / nbuf) & 1u, abort, p.wait_ns);
        if (q == 0) stamp_now(2);   // the first item buffer is built
        const long long seg_hi = min(hi, (long long)(item + 1) * tasks_per_expert);
        const uint4* bfrag = reinterpret_cast<const uint4*>(smem + sp.bfrag + buf * (nb * 512));
        const ulonglong2* da = reinterpret_cast<const ulonglong2*>(smem + sp.da + buf * (nb * 64));
        const int4* ci = reinterpret_cast<const int4*>(smem + sp.ci + buf * (nb * 128));
        const Item* its = reinterpret_cast<const Item*>(smem + sp.item + buf * 64);
        const int m = its->n_tok;
        const int g = lane >> 2, t4 = lane & 3;
        const bool narrow = m <= kNarrowTok && p.narrow;
        // the lane's two token columns, and in the narrow form the row group (of the pair) it finishes
        const int c0 = narrow ? 2 * (t4 & 1) : 2 * t4, c1 = c0 + 1, rn = t4 >> 1;
        const long long seg_lo = max(lo, (long long)item * tasks_per_expert);
        const int i_lo = int(seg_lo - lo), first = i_lo + (warp - i_lo % NW + NW) % NW;
        for (long long tau = lo + first; tau < seg_hi; tau += NW) {
            const int task = int(tau % tasks_per_expert);
            if constexpr (TASK4) {
                const int upc = units / cpt;
                float* o0 = nullptr;
                float* o1 = nullptr;
                if (m <= 2) {   // lane (g, t4) finishes row group t4 for tokens 0 and 1
                    uint64_t acc_lo = 0ull, acc_hi = 0ull;
                    for (int c = 0; c < cpt; ++c) {
                        const uint8_t* cp = chunk_wait();
                        units_mma_n2<UPC>(cp, quarter_bytes, upc, 2 * c * upc, bfrag, da, ci, lane, acc_lo, acc_hi);
                        chunk_done();
                    }
                    float sum[4];
                    unpack2(acc_lo, sum[0], sum[1]);
                    unpack2(acc_hi, sum[2], sum[3]);
                    const int grp = task * 4 + t4;
                    if (GATE_UP) {
                        const int row = grp * 8 + g;
                        p.gu[size_t(its->slot[0]) * p.ff + row] = make_float2(sum[0], sum[2]);
                        if (m > 1) p.gu[size_t(its->slot[1]) * p.ff + row] = make_float2(sum[1], sum[3]);
                    } else {
                        const int row = grp * 16 + g;
                        o0 = out_row(its->slot[0]);
                        put2(o0, row, sum[0], sum[2]);
                        if (m > 1) {
                            o1 = out_row(its->slot[1]);
                            put2(o1, row, sum[1], sum[3]);
                        }
                    }
                } else {        // two pairs in the narrow form: lanes t4 = 0, 1 finish the first group of a pair, 2, 3 the second
                    uint64_t acc_lo[2] = {0ull, 0ull}, acc_hi[2] = {0ull, 0ull};
                    for (int c = 0; c < cpt; ++c) {
                        const uint8_t* cp = chunk_wait();
                        units_mma_n4x2<UPC>(cp, quarter_bytes, upc, 2 * c * upc, bfrag, da, ci, lane, acc_lo, acc_hi);
                        chunk_done();
                    }
                    const int t0 = 2 * (t4 & 1), t1 = t0 + 1;
                    if (!GATE_UP) {
                        if (t0 < m) o0 = out_row(its->slot[t0]);
                        if (t1 < m) o1 = out_row(its->slot[t1]);
                    }
#pragma unroll
                    for (int pi = 0; pi < 2; ++pi) {
                        float sum[4];
                        unpack2(acc_lo[pi], sum[0], sum[1]);
                        unpack2(acc_hi[pi], sum[2], sum[3]);
                        const int grp = task * 4 + 2 * pi + (t4 >> 1);
                        if (GATE_UP) {
                            const int row = grp * 8 + g;
                            if (t0 < m) p.gu[size_t(its->slot[t0]) * p.ff + row] = make_float2(sum[0], sum[2]);
                            if (t1 < m) p.gu[size_t(its->slot[t1]) * p.ff + row] = make_float2(sum[1], sum[3]);
                        } else {
                            const int row = grp * 16 + g;
                            if (o0) put2(o0, row, sum[0], sum[2]);
                            if (o1) put2(o1, row, sum[1], sum[3]);
                        }
                    }
                }
            } else if (GATE_UP && narrow) {
                uint64_t acc_lo = 0ull, acc_hi = 0ull;   // {0.0f, 0.0f}
                const int upc = units / cpt;
                for (int c = 0; c < cpt; ++c) {
                    const uint8_t* cp = chunk_wait();
                    units_mma_narrow<UPC>(cp, half_bytes, upc, 2 * c * upc, bfrag, da, ci, lane, acc_lo, acc_hi);
                    chunk_done();
                }
                float sum[4];
                unpack2(acc_lo, sum[0], sum[1]);
                unpack2(acc_hi, sum[2], sum[3]);
                const int row = (task * 2 + rn) * 8 + g;
                if (c0 < m) p.gu[size_t(its->slot[c0]) * p.ff + row] = make_float2(sum[0], sum[2]);
                if (c1 < m) p.gu[size_t(its->slot[c1]) * p.ff + row] = make_float2(sum[1], sum[3]);
            } else if (!GATE_UP && narrow) {
                const int gpc = kDownGroups / cpt;   // groups per chunk
                float* o0 = nullptr;
                float* o1 = nullptr;
                if (c0 < m) o0 = out_row(its->slot[c0]);
                if (c1 < m) o1 = out_row(its->slot[c1]);
                for (int c = 0; c < cpt; ++c) {
                    const uint8_t* cp = chunk_wait();
#pragma unroll 1
                    for (int gd = 0; gd < gpc; gd += 2) {   // gpc is even
                        uint64_t acc_lo = 0ull, acc_hi = 0ull;
                        units_mma_narrow<UPC>(cp + size_t(gd) * group_bytes, group_bytes, units, 0, bfrag, da, ci, lane, acc_lo, acc_hi);
                        float sum[4];
                        unpack2(acc_lo, sum[0], sum[1]);
                        unpack2(acc_hi, sum[2], sum[3]);
                        const int row = ((task * cpt + c) * gpc + gd + rn) * 16 + g;
                        if (o0) put2(o0, row, sum[0], sum[2]);
                        if (o1) put2(o1, row, sum[1], sum[3]);
                    }
                    chunk_done();
                }
            } else if (GATE_UP) {
                uint64_t acc_lo[2] = {0ull, 0ull}, acc_hi[2] = {0ull, 0ull};   // {0.0f, 0.0f}
                const int upc = units / cpt;
                for (int c = 0; c < cpt; ++c) {
                    const uint8_t* cp = chunk_wait();
                    units_mma<UPC>(cp, half_bytes, upc, 2 * c * upc, bfrag, da, ci, lane, acc_lo, acc_hi);
                    chunk_done();
                }
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    float sum[4];
                    unpack2(acc_lo[r], sum[0], sum[1]);
                    unpack2(acc_hi[r], sum[2], sum[3]);
                    const int row = (task * 2 + r) * 8 + g;
                    if (c0 < m) p.gu[size_t(its->slot[c0]) * p.ff + row] = make_float2(sum[0], sum[2]);
                    if (c1 < m) p.gu[size_t(its->slot[c1]) * p.ff + row] = make_float2(sum[1], sum[3]);
                }
            } else {
                const int gpc = kDownGroups / cpt;   // groups per chunk
                for (int c = 0; c < cpt; ++c) {
                    const uint8_t* cp = chunk_wait();
#pragma unroll 1
                    for (int gd = 0; gd < gpc; gd += 2) {   // gpc is even
                        uint64_t acc_lo[2] = {0ull, 0ull}, acc_hi[2] = {0ull, 0ull};
                        units_mma<UPC>(cp + size_t(gd) * group_bytes, group_bytes, units, 0, bfrag, da, ci, lane, acc_lo, acc_hi);
                        float* o0 = nullptr;
                        float* o1 = nullptr;
                        if (c0 < m) o0 = out_row(its->slot[c0]);
                        if (c1 < m) o1 = out_row(its->slot[c1]);
#pragma unroll
                        for (int r = 0; r < 2; ++r) {
                            float sum[4];
                            unpack2(acc_lo[r], sum[0], sum[1]);
                            unpack2(acc_hi[r], sum[2], sum[3]);
                            const int row = ((task * cpt + c) * gpc + gd + r) * 16 + g;
                            if (o0) put2(o0, row, sum[0], sum[2]);
                            if (o1) put2(o1, row, sum[1], sum[3]);
                        }
                    }
                    chunk_done();
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(done + buf);
        if (q + ahead < nseg) {
            const int nxt = (q + ahead) % nbuf;   // the buffer of item q - 1
            if (q >= 1) mbar_wait_bounded(done + nxt, uint32_t((q - 1) / nbuf) & 1u, abort, p.wait_ns);
            build(q + ahead, ctid, NW * 32);
            __syncwarp();
            if (lane == 0) mbar_arrive(ready + nxt);
        }
    }
    __syncthreads();
    stamp_now(3);   // every warp of the block has finished
    if (*abort) {
        // A wait ran out: report it, and give copies still in flight time to land before the
        // block's shared memory is released.
        if (threadIdx.x == 0) p.status[0] = kDevWaitTimeout;
        const uint64_t t0 = global_ns();
        while (global_ns() - t0 < 2000000ull) {
        }
    }
}

// ---------------------------------------------------------------------------------------------
// The decode FFN as one kernel (items of at most kNarrowTok tokens): gate/up, then SwiGLU and the
// quantization of the hidden rows, then down, with one ring of weight chunks per warp that is never
// drained in between.
//   A block owns the same share of the gate/up tasks and of the down tasks (roughly the same
//   items). Its warps take the block's tasks round-robin over the whole sequence: first the gate/up
//   tasks in item order, then the down tasks. A gate/up task is two row groups in chunks of four
//   units of K, a down task four row groups in chunks of two units: the same 8 units = 4,608 bytes.
//   A warp that has finished its gate/up tasks of an item adds their number to the item's counter
//   (release). The hidden rows of an item are complete when its counter has reached the number of
//   gate/up tasks of an expert; whoever builds a down item waits for that (acquire, bounded), reads
//   the (gate x, up x) pairs of the item's slots, forms silu(gate x) * up x, quantizes it like
//   k_quant_hidden and writes codes, scales and accumulator inputs straight into the item buffer.
//   (Letting one warp build a whole item buffer, the first to get there, instead of all warps in
//   shares, was measured and is slower: the lone builder's global-memory round trips are serial.)
//   A block walks its down items starting from its second one: the first is shared with the block
//   before, which reaches it last in its own gate/up pass, the last is shared with the block after,
//   which took it first.
// Blocks wait for counters that other blocks raise, so every block must be resident: the grid is
// one block per SM (checked on the host), and every wait is bounded.
// Products, scaling and the order of additions are those of k_stream: the same bits.
constexpr int kMaxItemBufs4 = 4;                 // item buffers per half, at most
constexpr int kFfnBS = 16;                       // 16-byte vectors per block of the B fragments: token columns 0..3
constexpr uint32_t kFfnBfragBlock = kFfnBS * 16;
struct FfnPlan {
    uint32_t ring, g_bfrag, g_da, g_ci, g_item, d_bfrag, d_da, d_ci, d_item, bars, abort, total;
};
__host__ __device__ inline FfnPlan ffn_plan(int n, int ff, uint32_t chunk_bytes, int slots, int nbuf_g, int nbuf_d) {
    const uint32_t nbg = uint32_t(n / kQK), nbd = uint32_t(ff / kQK);
    FfnPlan s{};
    uint32_t off = 0;
    s.ring = off;
    off += uint32_t(slots) * chunk_bytes;
    off = (off + 127u) & ~127u;
    s.g_bfrag = off;
    off += uint32_t(nbuf_g) * nbg * kFfnBfragBlock;
    s.g_da = off;
    off += uint32_t(nbuf_g) * nbg * 64;
    s.g_ci = off;
    off += uint32_t(nbuf_g) * nbg * 128;
    s.g_item = off;
    off += uint32_t(nbuf_g) * 64;
    s.d_bfrag = off;
    off += uint32_t(nbuf_d) * nbd * kFfnBfragBlock;
    s.d_da = off;
    off += uint32_t(nbuf_d) * nbd * 64;
    s.d_ci = off;
    off += uint32_t(nbuf_d) * nbd * 128;
    s.d_item = off;
    off += uint32_t(nbuf_d) * 64;
    s.bars = off;          // `slots` ring barriers, then ready/done of the gate/up buffers, then of the down buffers
    off += uint32_t(slots + 4 * kMaxItemBufs4) * 8;
    off = (off + 15u) & ~15u;
    s.abort = off;
    off += 16;
    s.total = off;
    return s;
}
constexpr int kFfnUnitsGu = 4, kFfnUnitsDn = 2;   // units of K per chunk and row group
constexpr uint32_t kFfnChunkBytes = 2 * kFfnUnitsGu * kUnitBytes;
static_assert(kFfnChunkBytes == 4 * kFfnUnitsDn * kUnitBytes, "one ring slot serves both halves");

template <int NW>
__global__ void __launch_bounds__(NW * 32, 1) k_ffn(const StreamParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, ctid = threadIdx.x;
    const int nb_g = p.n / kQK, units_g = p.n / kUnitK, nb_d = p.ff / kQK, units_d = p.ff / kUnitK;
    const uint32_t gbytes_g = uint32_t(units_g) * kUnitBytes, gbytes_d = uint32_t(units_d) * kUnitBytes;   // one row group
    const int cpt_g = units_g / kFfnUnitsGu, cpt_d = units_d / kFfnUnitsDn, rpw = p.rpw;
    constexpr uint32_t chunk_bytes = kFfnChunkBytes, half_bytes = chunk_bytes / 2, quarter_bytes = chunk_bytes / 4;
    const int tpe_g = p.ff / 16, tpe_d = p.n / 64;   // tasks per expert
    const size_t section_d = size_t(p.ff / 8) * gbytes_g;   // the down rows follow the gate/up groups in a blob
    const int slots = NW * rpw, nbuf_g = p.nbuf, nbuf_d = p.nbuf_dn;
    const FfnPlan sp = ffn_plan(p.n, p.ff, chunk_bytes, slots, nbuf_g, nbuf_d);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + sp.bars);
    uint64_t* ready_g = bars + slots;
    uint64_t* done_g = ready_g + kMaxItemBufs4;
    uint64_t* ready_d = done_g + kMaxItemBufs4;
    uint64_t* done_d = ready_d + kMaxItemBufs4;
    uint64_t* full = bars + warp * rpw;                                   // this warp's ring barriers
    uint8_t* ring = smem + sp.ring + size_t(warp) * rpw * chunk_bytes;    // this warp's ring slots
    volatile int* abort = reinterpret_cast<volatile int*>(smem + sp.abort);
    if (threadIdx.x == 0) {
        for (int s = 0; s < slots; ++s) mbar_init(bars + s, 1);
        for (int b = 0; b < 4 * kMaxItemBufs4; ++b) mbar_init(ready_g + b, NW);
        *abort = 0;
        mbar_fence_init();
    }
    pdl_wait();   // the items, the counters (zeroed) and the quantized x are complete
    pdl_trigger();

    const int n_items = p.status[1];
    const long long tot_g = (long long)n_items * tpe_g, tot_d = (long long)n_items * tpe_d;
    const long long lo_g = tot_g * blockIdx.x / gridDim.x, hi_g = tot_g * (blockIdx.x + 1) / gridDim.x;
    const long long lo_d = tot_d * blockIdx.x / gridDim.x, hi_d = tot_d * (blockIdx.x + 1) / gridDim.x;
    const int nt_g = int(hi_g - lo_g), nt_d = int(hi_d - lo_d);
    if (nt_g + nt_d <= 0) return;   // uniform for the block
    // segments: runs of consecutive tasks of one item
    const int fi_g = nt_g > 0 ? int(lo_g / tpe_g) : 0, nseg_g = nt_g > 0 ? int((hi_g - 1) / tpe_g) - fi_g + 1 : 0;
    const int fi_d = nt_d > 0 ? int(lo_d / tpe_d) : 0, nseg_d = nt_d > 0 ? int((hi_d - 1) / tpe_d) - fi_d + 1 : 0;
    const int rot_d = nseg_d > 1 ? 1 : 0;
    const int ahead_g = nbuf_g - 1, ahead_d = nbuf_d - 1;
    __syncthreads();
    auto item_d = [&](int s) { return fi_d + (s + rot_d) % nseg_d; };   // the item of the s-th down segment in walking order
    auto seg_g = [&](int s, long long& a, int& len) {
        const long long it = fi_g + s;
        a = max(lo_g, it * tpe_g);
        len = int(min(hi_g, (it + 1) * tpe_g) - a);
    };
    auto seg_d = [&](int s, long long& a, int& len) {
        const long long it = item_d(s);
        a = max(lo_d, it * tpe_d);
        len = int(min(hi_d, (it + 1) * tpe_d) - a);
    };

    // ---- this warp's stream of chunks (lane 0 issues). The block's tasks are numbered through both
    // halves; task i belongs to warp i % NW. is_j: index of the task within its half.
    int is_ph = 0, is_s = -1, is_off = 0, is_len = 0, is_j = warp, is_c = 0, is_slot = 0, is_task = 0;
    long long is_a = 0;
    const uint8_t* is_blob = nullptr;
    auto is_seek = [&]() {   // to the segment that holds task is_j of half is_ph, or on to the next half; is_ph = 2: nothing left
        while (is_ph < 2) {
            if (is_s >= 0 && is_j < is_off + is_len) {
                is_task = int((is_a + (is_j - is_off)) % (is_ph ? tpe_d : tpe_g));
                return;
            }
            if (is_s + 1 < (is_ph ? nseg_d : nseg_g)) {
                ++is_s;
                is_off += is_len;
                if (is_ph) seg_d(is_s, is_a, is_len);
                else seg_g(is_s, is_a, is_len);
                is_blob = p.items[is_ph ? item_d(is_s) : fi_g + is_s].blob + (is_ph ? section_d : size_t(0));
            } else {
                ++is_ph;
                is_s = -1;
                is_off = 0;
                is_len = 0;
                is_j = ((warp - nt_g) % NW + NW) % NW;   // the first down task of this warp
            }
        }
    };
    auto issue_next = [&]() {   // lane 0 only
        if (is_ph >= 2) return;
        mbar_expect_tx(full + is_slot, chunk_bytes);
        uint8_t* dst = ring + size_t(is_slot) * chunk_bytes;
        int cpt;
        if (is_ph == 0) {   // the same K range of the task's two groups
            const uint8_t* src = is_blob + size_t(is_task) * (2 * gbytes_g) + size_t(is_c) * half_bytes;
            bulk_g2s(dst, src, half_bytes, full + is_slot);
            bulk_g2s(dst + half_bytes, src + gbytes_g, half_bytes, full + is_slot);
            cpt = cpt_g;
        } else {            // of the task's four groups
            const uint8_t* src = is_blob + size_t(is_task) * (4 * gbytes_d) + size_t(is_c) * quarter_bytes;
#pragma unroll
            for (int gq = 0; gq < 4; ++gq) bulk_g2s(dst + gq * quarter_bytes, src + size_t(gq) * gbytes_d, quarter_bytes, full + is_slot);
            cpt = cpt_d;
        }
        if (++is_slot == rpw) is_slot = 0;
        if (++is_c == cpt) {
            is_c = 0;
            is_j += NW;
            is_seek();
        }
    };
    if (lane == 0) {
        is_seek();
        for (int k = 0; k < rpw; ++k) issue_next();
    }
    int cs_slot = 0;
    uint32_t cs_phase = 0;
    auto chunk_wait = [&]() -> const uint8_t* {
        mbar_wait_bounded(full + cs_slot, cs_phase, abort, p.wait_ns);
        return ring + size_t(cs_slot) * chunk_bytes;
    };
    auto chunk_done = [&]() {
        __syncwarp();
        if (lane == 0) issue_next();
        if (++cs_slot == rpw) {
            cs_slot = 0;
            cs_phase ^= 1u;
        }
    };

    // ---- item buffers. gate/up: column g of the B fragments, scales and accumulator inputs <- the
    // quantized x row of the item's g-th token, in the narrow form (zeros in token columns 4..7, the
    // entries of lanes t4 = 2, 3 equal to those of t4 = 0, 1).
    auto build_x = [&](int s, int btid, int NT) {
        const Item* it = p.items + fi_g + s;
        const int buf = s % nbuf_g;
        uint32_t* bw = reinterpret_cast<uint32_t*>(smem + sp.g_bfrag + buf * (nb_g * kFfnBfragBlock));
        float* daw = reinterpret_cast<float*>(smem + sp.g_da + buf * (nb_g * 64));
        float* ciw = reinterpret_cast<float*>(smem + sp.g_ci + buf * (nb_g * 128));
        if (btid < kItemWords) reinterpret_cast<uint32_t*>(smem + sp.g_item + buf * 64)[btid] = reinterpret_cast<const uint32_t*>(it)[btid];
        const int m = min(it->n_tok, kNarrowTok);
        const int vpr = nb_g * 4;   // 16-byte vectors per row
        for (int base = btid; base < m * vpr; base += 4 * NT) {
            uint4 v[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int idx = base + k * NT;
                if (idx < m * vpr) {
                    const int g = idx / vpr, r = idx % vpr;
                    v[k] = reinterpret_cast<const uint4*>(p.aq + size_t(slot_token(it->slot[g], p.K, p.TK)) * p.n)[r];
                }
            }
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int idx = base + k * NT;
                if (idx < m * vpr) {
                    const int g = idx / vpr, r = idx % vpr;
                    reinterpret_cast<uint4*>(bw)[(r >> 2) * kFfnBS + g * 4 + (r & 3)] = v[k];
                }
            }
        }
        for (int idx = btid; idx < m * nb_g * 2; idx += NT) {
            const int g = idx / (nb_g * 2), r = idx % (nb_g * 2), b = r >> 1, h = r & 1;
            const size_t row = size_t(slot_token(it->slot[g], p.K, p.TK));
            const float av = p.aa[row * (nb_g * 2) + r], cv = p.ac[row * (nb_g * 2) + r];
            const int dst = (b * 4 + (g >> 1)) * 4 + h * 2 + (g & 1);
            daw[dst] = av;
            daw[dst + 8] = av;
            const float nv = narrow_bias(cv);
            const int cq = (b * 4 + (g >> 1)) * 8 + h * 2 + (g & 1);
            ciw[cq] = nv;
            ciw[cq + 16] = nv;
        }
    };
    // down: the same form from the item's hidden rows, which are made here from the (gate x, up x)
    // pairs. A thread owns four consecutive values, eight neighbouring lanes one 32-block.
    auto build_h = [&](int s, int btid, int NT) {
        const int item = item_d(s);
        const Item* it = p.items + item;
        const int buf = s % nbuf_d;
        if (lane == 0) {   // every gate/up task of the item has been counted
            const int* c = p.cnt + item;
            if (ld_acquire_gpu(c) < tpe_g && !*abort) {
                uint64_t t0 = 0;
                for (uint32_t polls = 1;; ++polls) {
                    if (ld_acquire_gpu(c) >= tpe_g) break;
                    __nanosleep(polls > 16 ? 200 : 40);
                    if ((polls & 31u) == 0) {
                        if (*abort) break;
                        const uint64_t now = global_ns();
                        if (t0 == 0) {
                            t0 = now;
                        } else if (now - t0 > p.wait_ns) {
                            *abort = 1;
                            break;
                        }
                    }
                }
            }
        }
        __syncwarp();
        uint32_t* bw = reinterpret_cast<uint32_t*>(smem + sp.d_bfrag + buf * (nb_d * kFfnBfragBlock));
        float* daw = reinterpret_cast<float*>(smem + sp.d_da + buf * (nb_d * 64));
        float* ciw = reinterpret_cast<float*>(smem + sp.d_ci + buf * (nb_d * 128));
        if (btid < kItemWords) reinterpret_cast<uint32_t*>(smem + sp.d_item + buf * 64)[btid] = reinterpret_cast<const uint32_t*>(it)[btid];
        build_hidden_narrow<kFfnBS>(p.gu, p.ff, it, bw, daw, ciw, btid, NT);
    };

    auto out_row = [&](int sl) -> float* { return sl >= p.TK ? p.ysh + size_t(sl - p.TK) * p.n : p.y + size_t(sl) * p.n; };
    auto put2 = [&](float* o, int row, float v0, float v8) {
        o[row] = v0;
        o[row + 8] = v8;
    };
    const int g = lane >> 2, t4 = lane & 3;

    // ---- gate/up
    if (ahead_g == 2 && nseg_g >= 2) {   // the first two items side by side, one half of the warps each
        constexpr int H = NW / 2;
        build_x(warp < H ? 0 : 1, warp < H ? ctid : ctid - H * 32, warp < H ? H * 32 : (NW - H) * 32);
        __syncwarp();
        if (lane == 0) {
            mbar_arrive(ready_g + 0);
            mbar_arrive(ready_g + 1);
        }
    } else {
        for (int q = 0; q < ahead_g && q < nseg_g; ++q) {
            build_x(q, ctid, NW * 32);
            __syncwarp();
            if (lane == 0) mbar_arrive(ready_g + q % nbuf_g);
        }
    }
    int off = 0;
    for (int s = 0; s < nseg_g; ++s) {
        const int buf = s % nbuf_g;
        mbar_wait_bounded(ready_g + buf, uint32_t(s / nbuf_g) & 1u, abort, p.wait_ns);
        long long a;
        int len;
        seg_g(s, a, len);
        const uint4* bfrag = reinterpret_cast<const uint4*>(smem + sp.g_bfrag + buf * (nb_g * kFfnBfragBlock));
        const ulonglong2* da = reinterpret_cast<const ulonglong2*>(smem + sp.g_da + buf * (nb_g * 64));
        const int4* ci = reinterpret_cast<const int4*>(smem + sp.g_ci + buf * (nb_g * 128));
        const Item* its = reinterpret_cast<const Item*>(smem + sp.g_item + buf * 64);
        const int m = its->n_tok;
        const int c0 = 2 * (t4 & 1), c1 = c0 + 1, rn = t4 >> 1;
        int mine = 0;
        for (int j = off + ((warp - off % NW) % NW + NW) % NW; j < off + len; j += NW) {
            const int task = int((a + (j - off)) % tpe_g);
            uint64_t acc_lo = 0ull, acc_hi = 0ull;
            for (int c = 0; c < cpt_g; ++c) {
                const uint8_t* cp = chunk_wait();
                units_mma_narrow<kFfnUnitsGu, kFfnBS>(cp, half_bytes, kFfnUnitsGu, 2 * c * kFfnUnitsGu, bfrag, da, ci, lane, acc_lo, acc_hi);
                chunk_done();
            }
            float sum[4];
            unpack2(acc_lo, sum[0], sum[1]);
            unpack2(acc_hi, sum[2], sum[3]);
            const int row = (task * 2 + rn) * 8 + g;
            if (c0 < m) p.gu[size_t(its->slot[c0]) * p.ff + row] = make_float2(sum[0], sum[2]);
            if (c1 < m) p.gu[size_t(its->slot[c1]) * p.ff + row] = make_float2(sum[1], sum[3]);
            ++mine;
        }
        off += len;
        __syncwarp();
        if (lane == 0) {
            if (mine) red_release_gpu_add(p.cnt + fi_g + s, mine);   // this warp's rows of the item are written
            mbar_arrive(done_g + buf);
        }
        if (s + ahead_g < nseg_g) {
            const int nxt = (s + ahead_g) % nbuf_g;   // the buffer of segment s - 1
            if (s >= 1) mbar_wait_bounded(done_g + nxt, uint32_t((s - 1) / nbuf_g) & 1u, abort, p.wait_ns);
            build_x(s + ahead_g, ctid, NW * 32);
            __syncwarp();
            if (lane == 0) mbar_arrive(ready_g + nxt);
        }
    }

    // ---- down (this warp's weight chunks of it are already on their way)
    for (int q = 0; q < ahead_d && q < nseg_d; ++q) {
        build_h(q, ctid, NW * 32);
        __syncwarp();
        if (lane == 0) mbar_arrive(ready_d + q % nbuf_d);
    }
    off = 0;
    for (int s = 0; s < nseg_d; ++s) {
        const int buf = s % nbuf_d;
        mbar_wait_bounded(ready_d + buf, uint32_t(s / nbuf_d) & 1u, abort, p.wait_ns);
        long long a;
        int len;
        seg_d(s, a, len);
        const uint4* bfrag = reinterpret_cast<const uint4*>(smem + sp.d_bfrag + buf * (nb_d * kFfnBfragBlock));
        const ulonglong2* da = reinterpret_cast<const ulonglong2*>(smem + sp.d_da + buf * (nb_d * 64));
        const int4* ci = reinterpret_cast<const int4*>(smem + sp.d_ci + buf * (nb_d * 128));
        const Item* its = reinterpret_cast<const Item*>(smem + sp.d_item + buf * 64);
        const int m = its->n_tok;
        for (int j = off + ((warp - (nt_g + off) % NW) % NW + NW) % NW; j < off + len; j += NW) {
            const int task = int((a + (j - off)) % tpe_d);
            if (m <= 2) {   // lane (g, t4) finishes row group t4 for tokens 0 and 1
                uint64_t acc_lo = 0ull, acc_hi = 0ull;
                for (int c = 0; c < cpt_d; ++c) {
                    const uint8_t* cp = chunk_wait();
                    units_mma_n2<kFfnUnitsDn, kFfnBS>(cp, quarter_bytes, kFfnUnitsDn, 2 * c * kFfnUnitsDn, bfrag, da, ci, lane, acc_lo, acc_hi);
                    chunk_done();
                }
                float sum[4];
                unpack2(acc_lo, sum[0], sum[1]);
                unpack2(acc_hi, sum[2], sum[3]);
                const int row = (task * 4 + t4) * 16 + g;
                put2(out_row(its->slot[0]), row, sum[0], sum[2]);
                if (m > 1) put2(out_row(its->slot[1]), row, sum[1], sum[3]);
            } else {        // two pairs in the narrow form: lanes t4 = 0, 1 finish the first group of a pair, 2, 3 the second
                uint64_t acc_lo[2] = {0ull, 0ull}, acc_hi[2] = {0ull, 0ull};
                for (int c = 0; c < cpt_d; ++c) {
                    const uint8_t* cp = chunk_wait();
                    units_mma_n4x2<kFfnUnitsDn, kFfnBS>(cp, quarter_bytes, kFfnUnitsDn, 2 * c * kFfnUnitsDn, bfrag, da, ci, lane, acc_lo, acc_hi);
                    chunk_done();
                }
                const int t0 = 2 * (t4 & 1), t1 = t0 + 1;
                float* o0 = t0 < m ? out_row(its->slot[t0]) : nullptr;
                float* o1 = t1 < m ? out_row(its->slot[t1]) : nullptr;
#pragma unroll
                for (int pi = 0; pi < 2; ++pi) {
                    float sum[4];
                    unpack2(acc_lo[pi], sum[0], sum[1]);
                    unpack2(acc_hi[pi], sum[2], sum[3]);
                    const int row = (task * 4 + 2 * pi + (t4 >> 1)) * 16 + g;
                    if (o0) put2(o0, row, sum[0], sum[2]);
                    if (o1) put2(o1, row, sum[1], sum[3]);
                }
            }
        }
        off += len;
        __syncwarp();
        if (lane == 0) mbar_arrive(done_d + buf);
        if (s + ahead_d < nseg_d) {
            const int nxt = (s + ahead_d) % nbuf_d;
            if (s >= 1) mbar_wait_bounded(done_d + nxt, uint32_t((s - 1) / nbuf_d) & 1u, abort, p.wait_ns);
            build_h(s + ahead_d, ctid, NW * 32);
            __syncwarp();
            if (lane == 0) mbar_arrive(ready_d + nxt);
        }
    }
    __syncthreads();
    if (*abort) {
        // A wait ran out: report it, and give copies still in flight time to land before the
        // block's shared memory is released.
        if (threadIdx.x == 0) p.status[0] = kDevWaitTimeout;
        const uint64_t t0 = global_ns();
        while (global_ns() - t0 < 2000000ull) {
        }
    }
}

// out[t] = sum over the token's slots in ascending expert id of w * y, then + ysh * sigmoid(gate).
// A thread owns four consecutive elements of one token. The order entries, the weights and the rows
// of eight slots at a time are loaded before the first addition (the loads do not depend on one
// another, the additions keep their order), so the kernel is three round trips to memory long
// instead of two per slot.
constexpr int kCombineElems = 4, kCombineBatch = 8;
__global__ void __launch_bounds__(256) k_combine_ordered(float* __restrict__ out, const float* __restrict__ y,
                                                         const float* __restrict__ wts, const int32_t* __restrict__ order,
                                                         const float* __restrict__ ysh, const float* __restrict__ gate, int n, int K,
                                                         int sh_lo, int sh_hi) {   // the shared expert's rows exist for tokens [sh_lo, sh_hi)
    const int i = (blockIdx.x * blockDim.x + threadIdx.x) * kCombineElems, t = blockIdx.y;   // n is a multiple of 128: four elements are all inside or all outside
    if (threadIdx.x == 0) {
        touch_l2(order + size_t(t) * K);
        touch_l2(wts);
        touch_l2(y);
        touch_l2(out + size_t(t) * n);
        if (ysh) touch_l2(ysh + size_t(t) * n);
    }
    pdl_wait();
    pdl_trigger();
    if (i >= n) return;
    float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    for (int k0 = 0; k0 < K; k0 += kCombineBatch) {
        int s[kCombineBatch];
        float w[kCombineBatch];
        float4 v[kCombineBatch];
#pragma unroll
        for (int j = 0; j < kCombineBatch; ++j) s[j] = k0 + j < K ? order[t * K + k0 + j] : -1;
#pragma unroll
        for (int j = 0; j < kCombineBatch; ++j)
            if (s[j] >= 0) {
                w[j] = wts[s[j]];
                v[j] = *reinterpret_cast<const float4*>(y + size_t(s[j]) * n + i);
            }
#pragma unroll
        for (int j = 0; j < kCombineBatch; ++j)
            if (s[j] >= 0) {
                acc.x = __fadd_rn(acc.x, __fmul_rn(w[j], v[j].x));
                acc.y = __fadd_rn(acc.y, __fmul_rn(w[j], v[j].y));
                acc.z = __fadd_rn(acc.z, __fmul_rn(w[j], v[j].z));
                acc.w = __fadd_rn(acc.w, __fmul_rn(w[j], v[j].w));
            }
    }
    if (ysh && t >= sh_lo && t < sh_hi) {
        const float g = gate ? sigmoid_ref(gate[t]) : 1.0f;
        const float4 v = *reinterpret_cast<const float4*>(ysh + size_t(t) * n + i);
        acc.x = __fadd_rn(acc.x, __fmul_rn(v.x, g));
        acc.y = __fadd_rn(acc.y, __fmul_rn(v.y, g));
        acc.z = __fadd_rn(acc.z, __fmul_rn(v.z, g));
        acc.w = __fadd_rn(acc.w, __fmul_rn(v.w, g));
    }
    *reinterpret_cast<float4*>(out + size_t(t) * n + i) = acc;
}

// ---- combine fused with the expert-parallel all-reduce over peer memory
// Layout of a rank's communication buffer: two slots of partial sums [max_T][n] fp32, then
// (256-byte aligned) flag words [FRX_EP_MAX_RANKS][kEpMaxBlocks] (word [q][b] is written by block b
// of rank q: the number of the last call whose partial sums that block has published), then local
// words: the number of calls completed, a ticket counter, and four cycle stamps of the last call.
constexpr int kEpMaxBlocks = FRX_EP_MAX_BLOCKS;
struct EpLayout {
    size_t slot_floats, flags, state, total;
};
__host__ __device__ inline EpLayout ep_layout(int max_T, int n) {
    EpLayout L{};
    L.slot_floats = size_t(max_T) * n;
    L.flags = align_up(2 * L.slot_floats * 4);
    L.state = L.flags + size_t(FRX_EP_MAX_RANKS) * kEpMaxBlocks * 4;
    L.total = L.state + 256;
    return L;
}
struct EpParams {
    int world, rank;
    float* partial[FRX_EP_MAX_RANKS];      // slot 0 of every rank's buffer
    uint32_t* flags[FRX_EP_MAX_RANKS];     // every rank's flag words
    uint32_t* state;                       // local: [0] calls completed so far, [1] ticket, [8..15] cycle stamps
    size_t slot_floats;
    unsigned long long wait_ns;
    int sh_lo, sh_hi;                      // this rank adds the shared expert's rows of tokens [sh_lo, sh_hi)
};
__device__ __forceinline__ void st_relaxed_sys(uint32_t* p, uint32_t v) { asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ void fence_acq_rel_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// out[t] = sum over ranks (in rank order) of that rank's partial sum; this rank's partial sum is
// what k_combine_ordered computes. A thread owns kEpElems output elements of one token, and their
// partial sums never leave its registers, so no barrier inside the GPU is needed. Block b stores
// its part into this rank's buffer and raises its own flag word at every peer (one thread per
// peer: system-scope fence, then the flag store), waits for block b of every peer (the only blocks
// whose data it reads; one thread per peer polls), then issues the loads of all peers' parts
// before the first addition, so the reads cost one NVLink round trip, and adds them in rank
// order: every rank gets the same bits. Blocks of different GPUs wait on one another, so all blocks
// of a launch must be resident at once: the host keeps the grid below the number of SMs times four.
// A slot is reused every other call, which is safe: a block sees a peer's flag of call c only
// after that peer's kernel of call c - 1 has ended (kernels of one stream run in order), i.e. after
// the peer has read everything of call c - 1.
constexpr int kEpElems = 4;   // consecutive elements per thread: one 16-byte access
__device__ __forceinline__ float4 ld_peer4(const float* p) {   // never from a cache of this GPU: the buffer is rewritten every other call
    float4 v;
    asm volatile("ld.relaxed.sys.global.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
    return v;
}
__global__ void __launch_bounds__(256) k_combine_allreduce(float* __restrict__ out, const float* __restrict__ y,
                                                           const float* __restrict__ wts, const int32_t* __restrict__ order,
                                                           const float* __restrict__ ysh, const float* __restrict__ gate, int n, int K,
                                                           const EpParams ep, int* __restrict__ status) {
    __shared__ int s_fail;
    pdl_wait();
    pdl_trigger();
    const int t = blockIdx.y;
    const int i = (blockIdx.x * 256 + threadIdx.x) * kEpElems;   // n is a multiple of 128: a thread's four elements are all inside or all outside
    const uint32_t bid = blockIdx.y * gridDim.x + blockIdx.x;
    const bool stamp = bid == 0 && threadIdx.x == 0;
    long long* stamps = reinterpret_cast<long long*>(ep.state + 8);
    const uint32_t call = ep.state[0] + 1;   // the same in every block: state[0] only changes after all blocks have read it
    const size_t slot = size_t(call & 1u) * ep.slot_floats;
    if (threadIdx.x == 0) s_fail = 0;
    if (stamp) stamps[0] = clock64();
    float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (i < n) {
        for (int k = 0; k < K; ++k) {
            const int s = order[t * K + k];
            if (s >= 0) {
                const float w = wts[s];
                const float4 v = *reinterpret_cast<const float4*>(y + size_t(s) * n + i);
                acc.x = __fadd_rn(acc.x, __fmul_rn(w, v.x));
                acc.y = __fadd_rn(acc.y, __fmul_rn(w, v.y));
                acc.z = __fadd_rn(acc.z, __fmul_rn(w, v.z));
                acc.w = __fadd_rn(acc.w, __fmul_rn(w, v.w));
            }
        }
        if (ysh && t >= ep.sh_lo && t < ep.sh_hi) {
            const float g = gate ? sigmoid_ref(gate[t]) : 1.0f;
            const float4 v = *reinterpret_cast<const float4*>(ysh + size_t(t) * n + i);
            acc.x = __fadd_rn(acc.x, __fmul_rn(v.x, g));
            acc.y = __fadd_rn(acc.y, __fmul_rn(v.y, g));
            acc.z = __fadd_rn(acc.z, __fmul_rn(v.z, g));
            acc.w = __fadd_rn(acc.w, __fmul_rn(v.w, g));
        }
        *reinterpret_cast<float4*>(ep.partial[ep.rank] + slot + size_t(t) * n + i) = acc;
    }
    // publish and wait, one thread per peer: the block's stores are ordered before these threads by
    // the block barrier; each makes them visible to the system, raises this block's flag at its
    // peer, and waits for the same block of that peer (flags only grow; the signed distance makes
    // wrap-around harmless)
    __syncthreads();
    if (stamp) stamps[1] = clock64();
    if (int(threadIdx.x) < ep.world && int(threadIdx.x) != ep.rank) {
        const int q = threadIdx.x;
        fence_acq_rel_sys();
        st_relaxed_sys(ep.flags[q] + size_t(ep.rank) * kEpMaxBlocks + bid, call);
        const uint32_t* theirs = ep.flags[ep.rank] + size_t(q) * kEpMaxBlocks + bid;
        uint64_t t0 = 0;
        uint32_t polls = 0;
        while (int32_t(ld_acquire_sys(theirs) - call) < 0) {
            if ((++polls & 63u) == 0) {
                const uint64_t now = global_ns();
                if (t0 == 0) {
                    t0 = now;
                } else if (now - t0 > ep.wait_ns) {
                    s_fail = 1;
                    break;
                }
            }
        }
    }
    __syncthreads();
    if (stamp) stamps[2] = clock64();
    if (s_fail) {
        if (threadIdx.x == 0) status[0] = kDevWaitTimeout;
    } else if (i < n) {
        float4 v[FRX_EP_MAX_RANKS];
#pragma unroll
        for (int q = 0; q < FRX_EP_MAX_RANKS; ++q)   // every peer's part is requested before any is used
            if (q < ep.world && q != ep.rank) v[q] = ld_peer4(ep.partial[q] + slot + size_t(t) * n + i);
        float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
        for (int q = 0; q < FRX_EP_MAX_RANKS; ++q) {
            if (q >= ep.world) break;
            const float4 a = q == ep.rank ? acc : v[q];
            if (q == 0) {
                sum = a;
            } else {
                sum.x = __fadd_rn(sum.x, a.x);
                sum.y = __fadd_rn(sum.y, a.y);
                sum.z = __fadd_rn(sum.z, a.z);
                sum.w = __fadd_rn(sum.w, a.w);
            }
        }
        *reinterpret_cast<float4*>(out + size_t(t) * n + i) = sum;
    }
    if (stamp) stamps[3] = clock64();
    // the call is complete on this rank once every block has passed its wait: a ticket counts
    // them and the last one advances the call number
    __syncthreads();
    if (threadIdx.x == 0) {
        const uint32_t blocks = gridDim.x * gridDim.y;
        if (atomicAdd(&ep.state[1], 1u) == blocks - 1) {
            ep.state[1] = 0;
            __threadfence();
            ep.state[0] = call;
        }
    }
}

// Expert-parallel prefill: this rank's part of the weighted sum, out[t] = sum over the token's
// slots whose expert is held here (e_map[id] >= 0), in ascending expert id, of w * y; tokens with
// no such slot get zeros (the rows are then summed over the ranks). One block per token.
__global__ void __launch_bounds__(256) k_combine_partial(float* __restrict__ out, const float* __restrict__ y, const float* __restrict__ wts,
                                                         const int32_t* __restrict__ ids, const int32_t* __restrict__ e_map, int n, int K) {
    __shared__ int s_slot[32];
    __shared__ float s_w[32];
    __shared__ int s_cnt;
    const int t = blockIdx.x;
    if (threadIdx.x == 0) s_cnt = 0;
    __syncthreads();
    if (int(threadIdx.x) < K) {
        const int k = threadIdx.x, e = ids[size_t(t) * K + k];
        if (e_map[e] >= 0) {
            int rank = 0;   // among the token's local slots, by expert id (then by k)
            for (int j = 0; j < K; ++j) {
                const int ej = ids[size_t(t) * K + j];
                if (e_map[ej] >= 0 && (ej < e || (ej == e && j < k))) ++rank;
            }
            s_slot[rank] = t * K + k;
            s_w[rank] = wts[size_t(t) * K + k];
            atomicAdd(&s_cnt, 1);
        }
    }
    __syncthreads();
    const int cnt = s_cnt;
    for (int i = threadIdx.x * 4; i < n; i += 256 * 4) {
        float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        for (int r = 0; r < cnt; ++r) {
            const float w = s_w[r];
            const float4 v = *reinterpret_cast<const float4*>(y + size_t(s_slot[r]) * n + i);
            acc.x = __fadd_rn(acc.x, __fmul_rn(w, v.x));
            acc.y = __fadd_rn(acc.y, __fmul_rn(w, v.y));
            acc.z = __fadd_rn(acc.z, __fmul_rn(w, v.z));
            acc.w = __fadd_rn(acc.w, __fmul_rn(w, v.w));
        }
        *reinterpret_cast<float4*>(out + size_t(t) * n + i) = acc;
    }
}

// k_moe_combine / k_stream_combine semantics: k order, as the hit list gives it
__global__ void __launch_bounds__(256) k_combine_hits(float* __restrict__ out, const float* __restrict__ yh,
                                                      const float* __restrict__ w, const int32_t* __restrict__ hit_n,
                                                      const float* __restrict__ shexp, const float* __restrict__ gate, int n, int K) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x, t = blockIdx.y;
    if (i >= n) return;
    const int kn = hit_n ? hit_n[t] : K;
    float acc = 0.0f;
    for (int k = 0; k < kn; ++k) acc = __fadd_rn(acc, __fmul_rn(w[t * K + k], yh[(size_t(t) * K + k) * n + i]));
    if (shexp) {
        const float g = gate ? sigmoid_ref(gate[t]) : 1.0f;
        acc = __fadd_rn(acc, __fmul_rn(shexp[size_t(t) * n + i], g));
    }
    out[size_t(t) * n + i] = acc;
}

// ---------------------------------------------------------------------------------------------
// moe_hits grouping: items from per-token lists of expert pointers. Slots s = t * K + k with
// k < hit_n[t] are live; live slots with the same pointer form one group (an expert several
// tokens hit is read once), groups ordered by first appearance, members in slot order.
// One block; S = T * K <= 1024.
__global__ void __launch_bounds__(1024) k_group_ptr(const uint8_t* const* __restrict__ hit_ptr, const int32_t* __restrict__ hit_n,
                                                    int T, int K, Item* __restrict__ items, int* __restrict__ status) {
    __shared__ const uint8_t* ptr[1024];
    __shared__ int scan[1024];
    const int s = threadIdx.x, S = T * K;
    if (s == 0 && status[3] != kCookie) {
        status[0] = kDevOk;
        status[2] = 0;
        status[3] = kCookie;
    }
    const bool live = s < S && (s % K) < hit_n[s / K];
    ptr[s] = live ? hit_ptr[s] : nullptr;
    __syncthreads();
    int leader = s, rank = 0, size = 0;
    if (live) {
        const uint8_t* mine = ptr[s];
        leader = -1;
        for (int j = 0; j < S; ++j)
            if (ptr[j] == mine) {
                if (leader < 0) leader = j;
                if (j < s) ++rank;
                ++size;
            }
    }
    const int my_items = (live && leader == s) ? (size + kTokPerItem - 1) / kTokPerItem : 0;
    scan[s] = my_items;
    __syncthreads();
    for (int o = 1; o < 1024; o <<= 1) {
        const int v = s >= o ? scan[s - o] : 0;
        __syncthreads();
        scan[s] += v;
        __syncthreads();
    }
    if (s == 0) status[1] = scan[1023];
    if (live) {
        const int base = scan[leader] - (size + kTokPerItem - 1) / kTokPerItem;   // exclusive offset of the group
        Item* it = items + base + rank / kTokPerItem;
        it->slot[rank % kTokPerItem] = s;
        if (rank % kTokPerItem == 0) {
            it->blob = ptr[s];
            it->expert = leader;
            const int m = min(kTokPerItem, size - rank);
            it->n_tok = m;
            for (int j = m; j < kTokPerItem; ++j) it->slot[j] = 0;
        }
    }
}

// one thread per item: its expert (binary search over item_off) and its slots
__global__ void __launch_bounds__(256) k_pf_items(const int* __restrict__ bounds, const int* __restrict__ item_off, int E,
                                                  const int32_t* __restrict__ perm, const uint8_t* __restrict__ experts, size_t stride,
                                                  const int* __restrict__ status, Item* __restrict__ items) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= status[1]) return;
    int lo = 0, hi = E;   // the e with item_off[e] <= i < item_off[e + 1]
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (item_off[mid] <= i) lo = mid; else hi = mid;
    }
    const int e = lo, base = bounds[e] + (i - item_off[e]) * kTokPerItem, m = min(kTokPerItem, bounds[e + 1] - base);
    Item it;
    it.blob = experts + size_t(e) * stride;
    it.expert = e;
    it.n_tok = m;
    for (int j = 0; j < kTokPerItem; ++j) it.slot[j] = j < m ? perm[base + j] : 0;
    items[i] = it;
}

// ---------------------------------------------------------------------------------------------

int g_nw = 16;   // consumer warps of k_stream (8, 12 or 16)
int g_narrow = 1; // items of at most kNarrowTok tokens take the narrow form of the inner product
int g_gu_chunks = 0;   // chunks per gate/up task (0: by shape)

struct StreamCfg {
    int nw_gu = 8, nw_dn = 8;     // warps per block
    int cpt_gu = 1, cpt_dn = 1;   // chunks per task
    int rpw_gu = 2, rpw_dn = 2;   // ring slots per warp
    int nbuf_gu = 2, nbuf_dn = 2; // item buffers
    uint32_t smem_gu = 0, smem_dn = 0;
};

// max_items: an upper bound of the work items of a launch when the caller knows one (decode), else
// 0. With few items most warps of a 16-warp block would have no task at all while the busy ones
// are limited by their two ring slots (a warp streams its task with only that much in flight):
// blocks of 4 or 8 warps with deeper rings serve small batches better.
// decode, when every item has at most four tokens: bit 0 = gate/up, bit 1 = down take tasks of four row groups
// (k_stream's TASK4 form). Measured at batch 64: down gains from it, gate/up does not.
int g_task4 = 2;
int g_evict_first = 1;  // decode: the weight copies carry an evict-first L2 policy (see l2_policy_evict_first)
int g_down_per_item = 256;   // weight of an item's buffer in down's split, in 1/16 of a task (measured best near 16 tasks: 102.4 us per layer against 103.5 with 0 and 106.5 with 1024)
int g_down_heavy = 22;  // decode: weight of a down task of an item of three or four tokens when the tasks are shared out (16 = as one of a smaller item, 0 = even split by count)
// decode: the hidden rows are formed and quantized inside down's item-buffer build (no k_quant_hidden launch)
// from this many tokens on. Measured (148 SMs, hidden 2048, 512 experts top-10): a gain of 2 to 3 us per layer
// at 4, 16 and 64 tokens, a loss of 3 to 4 us at 1 and 3 tokens, where the separate kernel's work runs on
// all SMs at once while down's weights are already on their way.
int g_fold_quant = 1, g_fold_min_tokens = 4;
// the weighted split of down's tasks costs the grouping kernel about 1 us: it pays from about 16 tokens on
constexpr int kSplitMinTokens = 16;
unsigned long long* g_stream_stamps = nullptr;   // measurement aid: see frx_debug_set_stream_stamps

int stream_cfg(int n, int ff, StreamCfg& c, long long max_items = 0, bool task4 = false) {
    const int budget = max_smem_optin() - 2048;   // less the kernels' static shared memory
    if (budget <= 0) return fail(FRX_ERR_CUDA, "no CUDA device");
    // a task is fetched as `chunks` chunks; the preferred warp count is kept if
    // every warp can have at least two ring slots (up to four), else fewer warps are used
    // and, first of all, three item buffers rather than two
    const int sms = sm_count();
    auto fit = [&](int kdim, uint32_t task_bytes, int chunks, long long max_tasks, int& nw, int& cpt, int& rpw, int& nbuf, uint32_t& bytes) {
        cpt = chunks;
        const uint32_t chunk = task_bytes / uint32_t(cpt);
        int first = task4 ? (g_nw >= 12 ? 16 : 8) : g_nw;
        if (max_tasks > 0 && max_tasks <= 4LL * sms) first = 4;
        else if (max_tasks > 0 && max_tasks <= 8LL * sms) first = 8;
        const int prefs[3] = {first, first > 16 ? 16 : first > 12 ? 12 : 8, 8};
        for (int k = 0; k < 3; ++k) {
            nw = prefs[k];
            for (nbuf = kMaxItemBufs; nbuf >= 2; --nbuf)
                for (rpw = nw <= 4 ? 8 : 4; rpw >= 2; --rpw) {
                    bytes = smem_plan(kdim, chunk, nw * rpw, nbuf).total;
                    if (int(bytes) <= budget) return true;
                }
        }
        return false;
    };
    const int gu_units = n / kUnitK, dn_units = ff / kUnitK;
    if (task4) {
        // a task is four groups, a chunk two units (or one) of K of all four: 4,608 bytes at the usual shapes
        const int gu_c = gu_units % 2 == 0 ? gu_units / 2 : gu_units, dn_c = dn_units % 2 == 0 ? dn_units / 2 : dn_units;
        if (!fit(n, uint32_t(gu_units) * kUnitBytes * 4, gu_c, max_items * (ff / 32), c.nw_gu, c.cpt_gu, c.rpw_gu, c.nbuf_gu, c.smem_gu) ||
            !fit(ff, uint32_t(dn_units) * kUnitBytes * 4, dn_c, max_items * (n / 64), c.nw_dn, c.cpt_dn, c.rpw_dn, c.nbuf_dn, c.smem_dn))
            return fail(FRX_ERR_SHAPE, "n %d / ff %d: tiles do not fit in shared memory", n, ff);
        auto round_nw = [](int nw) { return nw >= 12 ? 16 : nw >= 8 ? 8 : 4; };   // the forms that are built
        if (round_nw(c.nw_gu) != c.nw_gu || round_nw(c.nw_dn) != c.nw_dn) return fail(FRX_ERR_SHAPE, "unsupported warp count for four-group tasks");
        return FRX_OK;
    }
    // gate/up: a task is two groups, fetched in K slices; down: kDownGroups groups in two chunks of whole groups
    int gu_chunks = gu_units % 4 == 0 ? 4 : gu_units % 2 == 0 ? 2 : 1;
    if (g_gu_chunks > 0 && gu_units % g_gu_chunks == 0) gu_chunks = g_gu_chunks;
    if (!fit(n, uint32_t(gu_units) * kUnitBytes * 2, gu_chunks, max_items * (ff / 16), c.nw_gu, c.cpt_gu, c.rpw_gu, c.nbuf_gu, c.smem_gu) ||
        !fit(ff, uint32_t(dn_units) * kUnitBytes * kDownGroups, 2, max_items * (n / 16 / kDownGroups), c.nw_dn, c.cpt_dn, c.rpw_dn, c.nbuf_dn,
             c.smem_dn))
        return fail(FRX_ERR_SHAPE, "n %d / ff %d: tiles do not fit in shared memory", n, ff);
    return FRX_OK;
}

// The fused form (k_ffn): warps per block, ring slots per warp and item buffers that fit.
// Off by default: measured at batch 64 (148 SMs) the one kernel takes as long as the three it
// replaces (102 us against 57 + 9 + 39), and the chain of three overlaps better with its neighbours.
int g_fused = 0;
int g_ffn_nbuf_g = 0, g_ffn_nbuf_d = 0;   // > 0: that many item buffers (2 .. kMaxItemBufs4) instead of up to kMaxItemBufs, as fit
struct FfnCfg {
    int nw = 16, rpw = 2, nbuf_g = 2, nbuf_d = 2;
    uint32_t smem = 0;
};
bool ffn_cfg(int n, int ff, long long max_items, FfnCfg& c) {
    const int ug = n / kUnitK, ud = ff / kUnitK;
    if (ug % kFfnUnitsGu || ud % kFfnUnitsDn) return false;
    const int budget = max_smem_optin() - 2048, sms = sm_count();
    const long long max_tasks = max_items * (ff / 16);
    int first = g_nw >= 12 ? 16 : 8;
    if (max_tasks > 0 && max_tasks <= 4LL * sms) first = 4;
    else if (max_tasks > 0 && max_tasks <= 8LL * sms) first = 8;
    const int prefs[3] = {first, first > 8 ? 8 : first, 4};
    for (int k = 0; k < 3; ++k) {
        c.nw = prefs[k];
        for (c.nbuf_g = g_ffn_nbuf_g ? g_ffn_nbuf_g : kMaxItemBufs; c.nbuf_g >= 2; --c.nbuf_g)
            for (c.nbuf_d = g_ffn_nbuf_d ? g_ffn_nbuf_d : kMaxItemBufs; c.nbuf_d >= 2; --c.nbuf_d)
                for (c.rpw = c.nw <= 4 ? 8 : 4; c.rpw >= 2; --c.rpw) {
                    c.smem = ffn_plan(n, ff, kFfnChunkBytes, c.nw * c.rpw, c.nbuf_g, c.nbuf_d).total;
                    if (int(c.smem) <= budget) return true;
                }
    }
    return false;
}

template <bool GATE_UP, int NW>
void launch_stream_nw(const StreamParams& p, int upc, uint32_t smem, cudaStream_t stream) {
    const int sms = sm_count();
    constexpr int kFixed = 4;   // the benchmark shapes: n = 2048 in four chunks, ff = 512
    if (upc == kFixed)
        launch_pdl(k_stream<GATE_UP, NW, kFixed>, dim3(sms), dim3(NW * 32), smem, stream, p);
    else
        launch_pdl(k_stream<GATE_UP, NW, 0>, dim3(sms), dim3(NW * 32), smem, stream, p);   // any other split of K
}

template <bool GATE_UP>
void launch_stream4(const StreamParams& p, int nw, int upc, uint32_t smem, cudaStream_t stream) {
    const int sms = sm_count();
    auto go = [&](auto kernel, int threads) { launch_pdl(kernel, dim3(sms), dim3(threads), smem, stream, p); };
    if (upc == 2) {
        switch (nw) {
            case 4: go(k_stream<GATE_UP, 4, 2, true>, 128); break;
            case 8: go(k_stream<GATE_UP, 8, 2, true>, 256); break;
            default: go(k_stream<GATE_UP, 16, 2, true>, 512); break;
        }
    } else {
        switch (nw) {
            case 4: go(k_stream<GATE_UP, 4, 0, true>, 128); break;
            case 8: go(k_stream<GATE_UP, 8, 0, true>, 256); break;
            default: go(k_stream<GATE_UP, 16, 0, true>, 512); break;
        }
    }
}

template <bool GATE_UP>
void launch_stream(const StreamParams& p, int nw, int upc, uint32_t smem, cudaStream_t stream) {
    switch (nw) {
        case 4: launch_stream_nw<GATE_UP, 4>(p, upc, smem, stream); break;
        case 8: launch_stream_nw<GATE_UP, 8>(p, upc, smem, stream); break;
        case 12: launch_stream_nw<GATE_UP, 12>(p, upc, smem, stream); break;
        case 20: launch_stream_nw<GATE_UP, 20>(p, upc, smem, stream); break;
        default: launch_stream_nw<GATE_UP, 16>(p, upc, smem, stream); break;
    }
}

// The streaming kernels need more dynamic shared memory than the default limit. The attribute
// belongs to the function on one device, so it is set once per device that calls in.
int set_smem_attr() {
    static std::mutex mu;
    static bool done[64] = {};
    int dev = 0;
    FRX_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lk(mu);
    if (dev >= 0 && dev < 64 && done[dev]) return FRX_OK;
    const int lim = max_smem_optin() - 2048;   // dynamic part only: the kernels also hold a little static shared memory
    const void* fns[] = {
        reinterpret_cast<const void*>(k_stream<true, 4, 4>),   reinterpret_cast<const void*>(k_stream<true, 4, 0>),
        reinterpret_cast<const void*>(k_stream<false, 4, 4>),  reinterpret_cast<const void*>(k_stream<false, 4, 0>),
        reinterpret_cast<const void*>(k_stream<true, 8, 4>),   reinterpret_cast<const void*>(k_stream<true, 8, 0>),
        reinterpret_cast<const void*>(k_stream<false, 8, 4>),  reinterpret_cast<const void*>(k_stream<false, 8, 0>),
        reinterpret_cast<const void*>(k_stream<true, 12, 4>),  reinterpret_cast<const void*>(k_stream<true, 12, 0>),
        reinterpret_cast<const void*>(k_stream<false, 12, 4>), reinterpret_cast<const void*>(k_stream<false, 12, 0>),
        reinterpret_cast<const void*>(k_stream<true, 16, 4>),  reinterpret_cast<const void*>(k_stream<true, 16, 0>),
        reinterpret_cast<const void*>(k_stream<false, 16, 4>), reinterpret_cast<const void*>(k_stream<false, 16, 0>),
        reinterpret_cast<const void*>(k_stream<true, 20, 4>),  reinterpret_cast<const void*>(k_stream<true, 20, 0>),
        reinterpret_cast<const void*>(k_stream<false, 20, 4>), reinterpret_cast<const void*>(k_stream<false, 20, 0>),
        reinterpret_cast<const void*>(k_stream<true, 4, 2, true>),   reinterpret_cast<const void*>(k_stream<true, 4, 0, true>),
        reinterpret_cast<const void*>(k_stream<false, 4, 2, true>),  reinterpret_cast<const void*>(k_stream<false, 4, 0, true>),
        reinterpret_cast<const void*>(k_stream<true, 8, 2, true>),   reinterpret_cast<const void*>(k_stream<true, 8, 0, true>),
        reinterpret_cast<const void*>(k_stream<false, 8, 2, true>),  reinterpret_cast<const void*>(k_stream<false, 8, 0, true>),
        reinterpret_cast<const void*>(k_stream<true, 16, 2, true>),  reinterpret_cast<const void*>(k_stream<true, 16, 0, true>),
        reinterpret_cast<const void*>(k_stream<false, 16, 2, true>), reinterpret_cast<const void*>(k_stream<false, 16, 0, true>),
        reinterpret_cast<const void*>(k_ffn<4>), reinterpret_cast<const void*>(k_ffn<8>), reinterpret_cast<const void*>(k_ffn<16>)};
    for (const void* f : fns) FRX_CUDA(cudaFuncSetAttribute(f, cudaFuncAttributeMaxDynamicSharedMemorySize, lim));
    // the head kernel's grouping tables: 12 bytes per expert, 4 per slot, 52 per item (at most 4096 experts, 64 x 32 slots, 2064 items)
    const void* heads[] = {reinterpret_cast<const void*>(k_prologue<0>), reinterpret_cast<const void*>(k_prologue<4>),
                           reinterpret_cast<const void*>(k_prologue<16>), reinterpret_cast<const void*>(k_prologue<32>)};
    for (const void* f : heads) FRX_CUDA(cudaFuncSetAttribute(f, cudaFuncAttributeMaxDynamicSharedMemorySize, 168 * 1024));
    if (dev >= 0 && dev < 64) done[dev] = true;
    return FRX_OK;
}

struct ActBufs {
    int8_t* q;
    float* a;
    float* c;
};

// The expert FFN over the items of p: quantize x, gate/up + SwiGLU into p.h, quantize the
// hidden rows, down. x has x_rows rows of p.n values; p.h has h_rows rows of p.ff values.
// (The grouping kernel that fills p.items may be enqueued before or after the first quantizer.)
void launch_quant_x(const float* x, int x_rows, int n, const ActBufs& xb, cudaStream_t stream, int block64 = 0) {
    const size_t nblk = size_t(x_rows) * (n / kQ8);
    FRX_LAUNCH(kKQuant, stream, launch_pdl(k_quant_frag, dim3(unsigned((nblk * 8 + 255) / 256)), dim3(256), 0, stream, x, n, nblk, xb.q, xb.a, xb.c, block64));
}

void launch_ffn(StreamParams p, const ActBufs& xb, const ActBufs& hb, size_t h_rows, const StreamCfg& cfg, cudaStream_t stream,
                bool task4_gu = false, bool task4_dn = false, const FfnCfg* fused = nullptr, bool fold_quant = false) {
    p.narrow = g_narrow;
    p.wait_ns = wait_limit_ns();
    p.stamps = g_stream_stamps;
    if (fused) {   // one kernel for gate/up, the hidden rows and down (items of at most four tokens)
        p.aq = xb.q;
        p.aa = xb.a;
        p.ac = xb.c;
        p.rpw = fused->rpw;
        p.nbuf = fused->nbuf_g;
        p.nbuf_dn = fused->nbuf_d;
        p.cnt = p.status + kStatusWords;
        const dim3 grid(sm_count());
        switch (fused->nw) {
            case 4: FRX_LAUNCH(kKFfn, stream, launch_pdl(k_ffn<4>, grid, dim3(128), fused->smem, stream, p)); break;
            case 8: FRX_LAUNCH(kKFfn, stream, launch_pdl(k_ffn<8>, grid, dim3(256), fused->smem, stream, p)); break;
            default: FRX_LAUNCH(kKFfn, stream, launch_pdl(k_ffn<16>, grid, dim3(512), fused->smem, stream, p)); break;
        }
        return;
    }
    p.cpt = cfg.cpt_gu;
    p.rpw = cfg.rpw_gu;
    p.nbuf = cfg.nbuf_gu;
    p.aq = xb.q;
    p.aa = xb.a;
    p.ac = xb.c;
    if (task4_gu)
        FRX_LAUNCH(kKGateUp, stream, launch_stream4<true>(p, cfg.nw_gu, p.n / kUnitK / cfg.cpt_gu, cfg.smem_gu, stream));
    else
        FRX_LAUNCH(kKGateUp, stream, launch_stream<true>(p, cfg.nw_gu, p.n / kUnitK / cfg.cpt_gu, cfg.smem_gu, stream));
    // decode with items of at most four tokens: down makes the hidden rows itself, from gu
    p.from_gu = fold_quant && g_narrow && task4_dn && !p.row_list && !p.block64 ? 1 : 0;
    const size_t nblk = h_rows * (p.ff / kQ8);
    if (!p.from_gu)
        FRX_LAUNCH(kKQuant, stream, launch_pdl(k_quant_hidden, dim3(unsigned((nblk + 31) / 32)), dim3(256), 0, stream, (const float2*)p.gu, p.ff, nblk, p.h, hb.q, hb.a, hb.c, p.slot_ids, p.TK, p.e_lo, p.e_hi, p.block64, p.e_map, p.row_list, p.row_count, p.row_list ? 0 : 1));
    if (p.stamps) p.stamps += size_t(sm_count()) * 4;   // down's stamps follow gate/up's
    p.cpt = cfg.cpt_dn;
    p.rpw = cfg.rpw_dn;
    p.nbuf = cfg.nbuf_dn;
    p.aq = hb.q;
    p.aa = hb.a;
    p.ac = hb.c;
    if (task4_dn)
        FRX_LAUNCH(kKDown, stream, launch_stream4<false>(p, cfg.nw_dn, p.ff / kUnitK / cfg.cpt_dn, cfg.smem_dn, stream));
    else
        FRX_LAUNCH(kKDown, stream, launch_stream<false>(p, cfg.nw_dn, p.ff / kUnitK, cfg.smem_dn, stream));
}

template <class LayoutT>
ActBufs act_x(uint8_t* base, const LayoutT& L) {
    return ActBufs{reinterpret_cast<int8_t*>(base + L.xq), reinterpret_cast<float*>(base + L.xa), reinterpret_cast<float*>(base + L.xc)};
}
template <class LayoutT>
ActBufs act_h(uint8_t* base, const LayoutT& L) {
    return ActBufs{reinterpret_cast<int8_t*>(base + L.hq), reinterpret_cast<float*>(base + L.ha), reinterpret_cast<float*>(base + L.hc)};
}

int check_moe_shape(const char* who, int n, int ff, int K) {
    if (n < kUnitK || ff < kUnitK || n % kUnitK || ff % kUnitK || n > 8192 || ff > 8192)
        return fail(FRX_ERR_SHAPE, "%s: n %d and ff %d must be multiples of %d, at most 8192", who, n, ff, kUnitK);
    if (K < 1 || K > 32) return fail(FRX_ERR_SHAPE, "%s: K %d outside [1, 32]", who, K);
    return FRX_OK;
}

// The decode layer over T tokens, 64 at a time: head (route when `logits` is given, group,
// quantize x), gate/up + SwiGLU, quantize the hidden rows, down, combine. With `logits` the ids
// and weights are outputs, else inputs.
int decode_steps(const void* experts, size_t stride, int E, int e_lo, int e_hi, const void* shared, int n, int ff, const float* x,
                 const float* logits, int32_t* ids, float* wts, const float* gate_logit, int T, int K, float* out, float* yslot, void* ws,
                 size_t ws_bytes, cudaStream_t stream, const EpParams* ep = nullptr, int shared_t0 = 0, int shared_t1 = 1 << 30) {
    if (!experts || !x || !ids || !wts || !out || !ws) return fail(FRX_ERR_ARG, "frx_moe_decode: null pointer");
    if (T < 0 || E < 1 || E > 4096) return fail(FRX_ERR_ARG, "frx_moe_decode: T %d, E %d", T, E);
    if (e_lo < 0 || e_hi > E || e_lo > e_hi) return fail(FRX_ERR_ARG, "frx_moe_decode: expert range [%d, %d) outside [0, %d)", e_lo, e_hi, E);
    if (int rc = check_moe_shape("frx_moe_decode", n, ff, K)) return rc;
    if (logits && (E > 1024 || K > E)) return fail(FRX_ERR_SHAPE, "frx_moe_layer: unsupported router shape E %d, k %d", E, K);
    if ((uintptr_t(experts) | uintptr_t(shared) | stride) % 16 || uintptr_t(ws) % kAlign)
        return fail(FRX_ERR_ARG, "frx_moe_decode: experts, shared and stride must be 16-byte aligned, ws 256-byte aligned");
    if ((uintptr_t(out) | uintptr_t(yslot) | uintptr_t(x)) % 16) return fail(FRX_ERR_ARG, "frx_moe_decode: x, out and the per-slot output must be 16-byte aligned");
    if (stride < frx_q2_expert_bytes(n, ff)) return fail(FRX_ERR_ARG, "frx_moe_decode: stride %zu < blob %zu", stride, frx_q2_expert_bytes(n, ff));
    if (T == 0) return FRX_OK;
    const Layout L = make_layout(T, K, n, ff);
    if (ws_bytes < L.total) return fail(FRX_ERR_WORKSPACE, "frx_moe_decode: workspace %zu < %zu", ws_bytes, L.total);
    // with items cut at four tokens either streaming kernel may take tasks of four row groups
    const bool task4_gu = g_narrow && (g_task4 & 1), task4_dn = g_narrow && (g_task4 & 2);
    StreamCfg cfg;
    if (int rc = stream_cfg(n, ff, cfg, L.max_items, false)) return rc;   // max_items: the most items a chunk of tokens can make
    if (task4_gu || task4_dn) {
        StreamCfg c4;
        if (int rc = stream_cfg(n, ff, c4, L.max_items, true)) return rc;
        if (task4_gu) {
            cfg.nw_gu = c4.nw_gu;
            cfg.cpt_gu = c4.cpt_gu;
            cfg.rpw_gu = c4.rpw_gu;
            cfg.nbuf_gu = c4.nbuf_gu;
            cfg.smem_gu = c4.smem_gu;
        }
        if (task4_dn) {
            cfg.nw_dn = c4.nw_dn;
            cfg.cpt_dn = c4.cpt_dn;
            cfg.rpw_dn = c4.rpw_dn;
            cfg.nbuf_dn = c4.nbuf_dn;
            cfg.smem_dn = c4.smem_dn;
        }
    }
    if (int rc = set_smem_attr()) return rc;
    FfnCfg fcfg;
    const bool fused = g_fused && g_narrow && ffn_cfg(n, ff, L.max_items, fcfg);
    auto* base = static_cast<uint8_t*>(ws);
    int* status = reinterpret_cast<int*>(base + L.status);
    Item* items = reinterpret_cast<Item*>(base + L.items);
    int32_t* order = reinterpret_cast<int32_t*>(base + L.order);
    const int sms = sm_count();

    for (int t0 = 0; t0 < T; t0 += kMaxChunkTokens) {
        const int Tc = T - t0 < kMaxChunkTokens ? T - t0 : kMaxChunkTokens;
        const ActBufs xb = act_x(base, L);
        // the tokens of this chunk that get the shared expert here
        const int sh_lo = std::min(std::max(shared_t0 - t0, 0), Tc), sh_hi = std::max(std::min(shared_t1 - t0, Tc), sh_lo);
        const size_t nblk = size_t(Tc) * (n / kQ8);
        const unsigned want = unsigned(std::min<size_t>((nblk + 127) / 128, size_t(sms)));   // a block of 1024 threads quantizes 128 blocks of 32 values per pass
        const unsigned qblocks = (want + kHeadCluster - 1) / kHeadCluster * kHeadCluster;
        // the down kernel's tasks are shared out by weight when every item is narrow (see DownSplit)
        DownSplit split{nullptr, sms, n / 64, g_down_heavy, g_down_per_item};
        if (g_narrow && g_down_heavy > 0 && Tc >= kSplitMinTokens && L.max_items <= 1024 && sms <= kMaxStreamBlocks) split.ranges = reinterpret_cast<int*>(base + L.ranges);
        const size_t dyn = size_t(E) * 8 + size_t(Tc) * K * 4 + (split.ranges ? size_t(L.max_items) * 4 : 0) + size_t(E) * 4 + 16 +
                           size_t(L.max_items) * sizeof(Item);
        auto head = [&](auto kernel) {
            return launch_pdl_cluster(kernel, dim3(kHeadCluster + qblocks), dim3(1024), dyn, stream, kHeadCluster, logits ? logits + size_t(t0) * E : (const float*)nullptr,
                              ids + size_t(t0) * K, wts + size_t(t0) * K, Tc, K, E, e_lo, e_hi, static_cast<const uint8_t*>(experts), stride,
                              static_cast<const uint8_t*>(shared), items, status, order, L.max_items, x + size_t(t0) * n, n, nblk, xb.q, xb.a,
                              xb.c, g_narrow ? kNarrowTok : kTokPerItem, split, sh_lo, sh_hi,
                              g_stream_stamps ? g_stream_stamps + size_t(sms) * 8 : (unsigned long long*)nullptr);
        };
        if (!logits)
            FRX_LAUNCH(kKPrologue, stream, head(k_prologue<0>));
        else if (E <= 128)
            FRX_LAUNCH(kKPrologue, stream, head(k_prologue<4>));
        else if (E <= 512)
            FRX_LAUNCH(kKPrologue, stream, head(k_prologue<16>));
        else
            FRX_LAUNCH(kKPrologue, stream, head(k_prologue<32>));
        StreamParams p{};
        p.items = items;
        p.status = status;
        p.gu = reinterpret_cast<float2*>(base + L.gu);
        p.h = reinterpret_cast<float*>(base + L.h);
        p.y = yslot ? yslot + size_t(t0) * K * n : reinterpret_cast<float*>(base + L.y);
        p.ysh = reinterpret_cast<float*>(base + L.ysh);
        p.n = n;
        p.ff = ff;
        p.K = K;
        p.TK = Tc * K;
        p.ranges = split.ranges;
        p.stream_once = g_evict_first;
        if (e_lo > 0 || e_hi < E) {
            p.slot_ids = ids + size_t(t0) * K;
            p.e_lo = e_lo;
            p.e_hi = e_hi;
        }
        launch_ffn(p, xb, act_h(base, L), size_t(Tc) * K + (shared ? Tc : 0), cfg, stream, task4_gu, task4_dn, fused ? &fcfg : nullptr, g_fold_quant && Tc >= g_fold_min_tokens);
        if (ep) {   // one chunk only (the caller checked T <= 64)
            EpParams epc = *ep;
            epc.sh_lo = sh_lo;
            epc.sh_hi = sh_hi;
            FRX_LAUNCH(kKCombine, stream, launch_pdl(k_combine_allreduce, dim3((n + 256 * kEpElems - 1) / (256 * kEpElems), Tc), dim3(256), 0, stream, out,
                                                            (const float*)p.y, (const float*)wts, (const int32_t*)order,
                                                            (const float*)(shared ? p.ysh : nullptr), gate_logit, n, K, epc, status));
        } else
            FRX_LAUNCH(kKCombine, stream, launch_pdl(k_combine_ordered, dim3((n + 256 * kCombineElems - 1) / (256 * kCombineElems), Tc), dim3(256), 0, stream, out + size_t(t0) * n, (const float*)p.y,
                                                            (const float*)(wts + size_t(t0) * K), (const int32_t*)order, (const float*)(shared ? p.ysh : nullptr),
                                                            gate_logit ? gate_logit + t0 : (const float*)nullptr, n, K, sh_lo, sh_hi));
    }
    FRX_CUDA(cudaGetLastError());
    return FRX_OK;
}

}  // namespace
}  // namespace frx

using namespace frx;

extern "C" {

int frx_quantize_q8(frx_stream_t stream, const float* x, int T, int n, int8_t* q, float* d) {
    if (T < 0 || n < kQ8 || n % kQ8) return fail(FRX_ERR_SHAPE, "frx_quantize_q8: T %d, n %d", T, n);
    if (T == 0) return FRX_OK;   // an empty batch: nothing to do, pointers may be null
    if (!x || !q || !d) return fail(FRX_ERR_ARG, "frx_quantize_q8: null pointer");
    const size_t nblk = size_t(T) * (n / kQ8);
    if (uintptr_t(x) % 16 == 0 && uintptr_t(q) % 4 == 0)
        FRX_LAUNCH(kKQuant, stream, k_quant_q8_quads<<<unsigned((nblk * 8 + 255) / 256), 256, 0, stream>>>(x, nblk, q, d));
    else
        FRX_LAUNCH(kKQuant, stream, k_quant_q8<<<unsigned((nblk + 7) / 8), 256, 0, stream>>>(x, nblk, q, d, nullptr));
    FRX_CUDA(cudaGetLastError());
    return FRX_OK;
}

size_t frx_moe_decode_workspace_bytes(int T, int K, int n, int ff) {
    if (T < 1 || K < 1 || n < kUnitK || ff < kUnitK) return 0;
    return make_layout(T, K, n, ff).total;
}

int frx_moe_decode(const void* experts, size_t stride, int E, const void* shared, int n, int ff, const float* x,
                   const int32_t* ids, const float* wts, const float* gate_logit, int T, int K, float* out, float* yslot,
                   void* ws, size_t ws_bytes, frx_stream_t stream) {
    return frx_moe_decode_ep(experts, stride, E, 0, E, shared, n, ff, x, ids, wts, gate_logit, T, K, out, yslot, ws, ws_bytes, stream);
}

int frx_moe_decode_ep(const void* experts, size_t stride, int E, int e_lo, int e_hi, const void* shared, int n, int ff,
                      const float* x, const int32_t* ids, const float* wts, const float* gate_logit, int T, int K, float* out,
                      float* yslot, void* ws, size_t ws_bytes, frx_stream_t stream) {
    if (!ids || !wts) return fail(FRX_ERR_ARG, "frx_moe_decode: null pointer");
    return decode_steps(experts, stride, E, e_lo, e_hi, shared, n, ff, x, nullptr, const_cast<int32_t*>(ids), const_cast<float*>(wts),
                        gate_logit, T, K, out, yslot, ws, ws_bytes, stream);
}

size_t frx_moe_layer_workspace_bytes(int T, int K, int n, int ff) {
    const size_t d = frx_moe_decode_workspace_bytes(T, K, n, ff);
    if (!d) return 0;
    return d + 2 * align_up(size_t(T) * K * 4);
}

int frx_moe_layer(const void* experts, size_t stride, int E, const void* shared, int n, int ff, const float* x,
                  const float* logits, const float* gate_logit, int T, int K, float* out, int32_t* ids_out, float* wts_out,
                  void* ws, size_t ws_bytes, frx_stream_t stream) {
    return frx_moe_layer_ep(experts, stride, E, 0, E, shared, n, ff, x, logits, gate_logit, T, K, out, ids_out, wts_out, ws, ws_bytes, stream);
}

int frx_moe_layer_ep(const void* experts, size_t stride, int E, int e_lo, int e_hi, const void* shared, int n, int ff, const float* x,
                     const float* logits, const float* gate_logit, int T, int K, float* out, int32_t* ids_out, float* wts_out,
                     void* ws, size_t ws_bytes, frx_stream_t stream) {
    if (!logits || !ws) return fail(FRX_ERR_ARG, "frx_moe_layer: null pointer");
    if (int rc = check_moe_shape("frx_moe_layer", n, ff, K)) return rc;
    if (T < 0) return fail(FRX_ERR_ARG, "frx_moe_layer: T %d", T);
    if (T == 0) return FRX_OK;
    const size_t d = frx_moe_decode_workspace_bytes(T, K, n, ff), r = align_up(size_t(T) * K * 4);
    if (ws_bytes < d + 2 * r) return fail(FRX_ERR_WORKSPACE, "frx_moe_layer: workspace %zu < %zu", ws_bytes, d + 2 * r);
    auto* base = static_cast<uint8_t*>(ws);
    int32_t* ids = ids_out ? ids_out : reinterpret_cast<int32_t*>(base + d);
    float* wts = wts_out ? wts_out : reinterpret_cast<float*>(base + d + r);
    return decode_steps(experts, stride, E, e_lo, e_hi, shared, n, ff, x, logits, ids, wts, gate_logit, T, K, out, nullptr, ws, d, stream);
}

size_t frx_ep_flags_offset(int max_T, int n) {
    if (max_T < 1 || n < 1) return 0;
    return ep_layout(max_T, n).flags;
}

size_t frx_ep_buffer_bytes(int max_T, int n) {
    if (max_T < 1 || n < 1) return 0;
    return ep_layout(max_T, n).total;
}

int frx_ep_buffer_create(void** buffer, int max_T, int n) {
    if (!buffer || max_T < 1 || n < 1) return fail(FRX_ERR_ARG, "frx_ep_buffer_create: bad argument");
    const size_t bytes = ep_layout(max_T, n).total;
    void* p = nullptr;
    FRX_CUDA(cudaMalloc(&p, bytes));   // its own allocation: CUDA IPC exports whole allocations
    cudaError_t e = cudaMemset(p, 0, bytes);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
        cudaFree(p);
        return cuda_fail(e, "frx_ep_buffer_create: cudaMemset");
    }
    *buffer = p;
    return FRX_OK;
}

int frx_ep_buffer_destroy(void* buffer) {
    if (buffer) FRX_CUDA(cudaFree(buffer));
    return FRX_OK;
}

int frx_ipc_export(const void* buffer, void* handle) {
    static_assert(sizeof(cudaIpcMemHandle_t) == FRX_IPC_HANDLE_BYTES, "handle size");
    if (!buffer || !handle) return fail(FRX_ERR_ARG, "frx_ipc_export: null pointer");
    cudaIpcMemHandle_t h;
    FRX_CUDA(cudaIpcGetMemHandle(&h, const_cast<void*>(buffer)));
    std::memcpy(handle, &h, sizeof h);
    return FRX_OK;
}

int frx_ipc_open(const void* handle, void** mapped) {
    if (!handle || !mapped) return fail(FRX_ERR_ARG, "frx_ipc_open: null pointer");
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle, sizeof h);
    FRX_CUDA(cudaIpcOpenMemHandle(mapped, h, cudaIpcMemLazyEnablePeerAccess));
    return FRX_OK;
}

int frx_ipc_close(void* mapped) {
    if (mapped) FRX_CUDA(cudaIpcCloseMemHandle(mapped));
    return FRX_OK;
}

int frx_moe_layer_ep_allreduce(const void* experts, size_t stride, int E, int e_lo, int e_hi, const void* shared, int n, int ff,
                               const float* x, const float* logits, const float* gate_logit, int T, int K, float* out,
                               int32_t* ids_out, float* wts_out, const frx_ep_comm* comm, void* ws, size_t ws_bytes,
                               frx_stream_t stream) {
    return frx_moe_layer_ep_allreduce_dealt(experts, stride, E, e_lo, e_hi, shared, 0, T, n, ff, x, logits, gate_logit, T, K, out, ids_out, wts_out,
                                            comm, ws, ws_bytes, stream);
}

int frx_moe_layer_ep_allreduce_dealt(const void* experts, size_t stride, int E, int e_lo, int e_hi, const void* shared, int shared_t0,
                                     int shared_t1, int n, int ff, const float* x, const float* logits, const float* gate_logit, int T, int K,
                                     float* out, int32_t* ids_out, float* wts_out, const frx_ep_comm* comm, void* ws, size_t ws_bytes,
                                     frx_stream_t stream) {
    if (!logits || !ws || !comm) return fail(FRX_ERR_ARG, "frx_moe_layer_ep_allreduce: null pointer");
    if (shared && (shared_t0 < 0 || shared_t1 > T || shared_t0 > shared_t1))
        return fail(FRX_ERR_ARG, "frx_moe_layer_ep_allreduce: shared-expert tokens [%d, %d) outside [0, %d)", shared_t0, shared_t1, T);
    if (comm->world < 1 || comm->world > FRX_EP_MAX_RANKS || comm->rank < 0 || comm->rank >= comm->world)
        return fail(FRX_ERR_ARG, "frx_moe_layer_ep_allreduce: rank %d of %d", comm->rank, comm->world);
    if (T < 0 || T > kMaxChunkTokens || T > comm->max_T || n != comm->n)
        return fail(FRX_ERR_SHAPE, "frx_moe_layer_ep_allreduce: T %d (at most %d and the buffers' %d), n %d (buffers' %d)", T, kMaxChunkTokens,
                    comm->max_T, n, comm->n);
    if (int rc = check_moe_shape("frx_moe_layer_ep_allreduce", n, ff, K)) return rc;
    if (uintptr_t(out) % 16) return fail(FRX_ERR_ARG, "frx_moe_layer_ep_allreduce: out must be 16-byte aligned");
    if (T == 0) return FRX_OK;   // every rank skips the call alike
    // blocks of different GPUs wait on one another: all of a launch must be resident at once
    const long long blocks = (long long)((n + 256 * kEpElems - 1) / (256 * kEpElems)) * T;
    if (blocks > 4LL * sm_count() || blocks > kEpMaxBlocks)
        return fail(FRX_ERR_SHAPE, "frx_moe_layer_ep_allreduce: %lld blocks would not be resident together", blocks);
    const EpLayout L = ep_layout(comm->max_T, comm->n);
    EpParams ep{};
    ep.world = comm->world;
    ep.rank = comm->rank;
    for (int q = 0; q < comm->world; ++q) {
        if (!comm->buffer[q]) return fail(FRX_ERR_ARG, "frx_moe_layer_ep_allreduce: buffer of rank %d is null", q);
        ep.partial[q] = static_cast<float*>(comm->buffer[q]);
        ep.flags[q] = reinterpret_cast<uint32_t*>(static_cast<uint8_t*>(comm->buffer[q]) + L.flags);
    }
    ep.state = reinterpret_cast<uint32_t*>(static_cast<uint8_t*>(comm->buffer[comm->rank]) + L.state);
    ep.slot_floats = L.slot_floats;
    ep.wait_ns = wait_limit_ns();
    const size_t d = frx_moe_decode_workspace_bytes(T, K, n, ff), r = align_up(size_t(T) * K * 4);
    if (ws_bytes < d + 2 * r) return fail(FRX_ERR_WORKSPACE, "frx_moe_layer_ep_allreduce: workspace %zu < %zu", ws_bytes, d + 2 * r);
    auto* base = static_cast<uint8_t*>(ws);
    int32_t* ids = ids_out ? ids_out : reinterpret_cast<int32_t*>(base + d);
    float* wts = wts_out ? wts_out : reinterpret_cast<float*>(base + d + r);
    return decode_steps(experts, stride, E, e_lo, e_hi, shared, n, ff, x, logits, ids, wts, gate_logit, T, K, out, nullptr, ws, d, stream, &ep,
                        shared_t0, shared_t1);
}

int frx_ep_debug_stamps(const void* own_buffer, int max_T, int n, long long* cycles4) {
    if (!own_buffer || !cycles4 || max_T < 1 || n < 1) return fail(FRX_ERR_ARG, "frx_ep_debug_stamps: bad argument");
    const EpLayout L = ep_layout(max_T, n);
    FRX_CUDA(cudaMemcpy(cycles4, static_cast<const uint8_t*>(own_buffer) + L.state + 32, 4 * sizeof(long long), cudaMemcpyDeviceToHost));
    return FRX_OK;
}

size_t frx_moe_layer_host_workspace_bytes(int T, int K, int n, int ff, int E) {
    const size_t l = frx_moe_layer_workspace_bytes(T, K, n, ff);
    if (!l || E < 1) return 0;
    return l + align_up(size_t(T) * n * 4) * 2 + align_up(size_t(T) * E * 4) + align_up(size_t(T) * 4);
}

int frx_moe_layer_host(const void* experts, size_t stride, int E, const void* shared, int n, int ff, const float* x_host,
                       const float* logits_host, const float* gate_logit_host, int T, int K, float* out_host, void* ws,
                       size_t ws_bytes, frx_stream_t stream) {
    if (!x_host || !logits_host || !out_host || !ws) return fail(FRX_ERR_ARG, "frx_moe_layer_host: null pointer");
    if (int rc = check_moe_shape("frx_moe_layer_host", n, ff, K)) return rc;
    if (T < 1 || E < 1) return fail(FRX_ERR_ARG, "frx_moe_layer_host: T %d, E %d", T, E);
    const size_t need = frx_moe_layer_host_workspace_bytes(T, K, n, ff, E);
    if (ws_bytes < need) return fail(FRX_ERR_WORKSPACE, "frx_moe_layer_host: workspace %zu < %zu", ws_bytes, need);
    const size_t l = frx_moe_layer_workspace_bytes(T, K, n, ff);
    auto* base = static_cast<uint8_t*>(ws);
    float* dx = reinterpret_cast<float*>(base + l);
    float* dout = reinterpret_cast<float*>(base + l + align_up(size_t(T) * n * 4));
    float* dlog = reinterpret_cast<float*>(base + l + 2 * align_up(size_t(T) * n * 4));
    float* dgate = reinterpret_cast<float*>(base + l + 2 * align_up(size_t(T) * n * 4) + align_up(size_t(T) * E * 4));
    FRX_CUDA(cudaMemcpyAsync(dx, x_host, size_t(T) * n * 4, cudaMemcpyHostToDevice, stream));
    FRX_CUDA(cudaMemcpyAsync(dlog, logits_host, size_t(T) * E * 4, cudaMemcpyHostToDevice, stream));
    if (gate_logit_host) FRX_CUDA(cudaMemcpyAsync(dgate, gate_logit_host, size_t(T) * 4, cudaMemcpyHostToDevice, stream));
    if (int rc = frx_moe_layer(experts, stride, E, shared, n, ff, dx, dlog, gate_logit_host ? dgate : nullptr, T, K, dout, nullptr,
                               nullptr, ws, l, stream))
        return rc;
    FRX_CUDA(cudaMemcpyAsync(out_host, dout, size_t(T) * n * 4, cudaMemcpyDeviceToHost, stream));
    FRX_CUDA(cudaStreamSynchronize(stream));
    return FRX_OK;
}

namespace {
constexpr int kHostSlots = 4;   // staging slots of frx_moe_layers_host
struct HostPipe {
    cudaStream_t in = nullptr, out = nullptr;
    cudaEvent_t start = nullptr, copied[kHostSlots] = {}, computed[kHostSlots] = {}, returned[kHostSlots] = {};
};
// The copy streams and events of the current device, created at the first call.
int host_pipe(HostPipe** pipe) {
    static std::mutex mu;
    static HostPipe pipes[64];
    int dev = 0;
    FRX_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(FRX_ERR_ARG, "frx_moe_layers_host: device ordinal %d not supported", dev);
    std::lock_guard<std::mutex> lk(mu);
    HostPipe& hp = pipes[dev];
    if (!hp.in) {
        FRX_CUDA(cudaStreamCreateWithFlags(&hp.in, cudaStreamNonBlocking));
        FRX_CUDA(cudaStreamCreateWithFlags(&hp.out, cudaStreamNonBlocking));
        FRX_CUDA(cudaEventCreateWithFlags(&hp.start, cudaEventDisableTiming));
        for (int i = 0; i < kHostSlots; ++i) {
            FRX_CUDA(cudaEventCreateWithFlags(&hp.copied[i], cudaEventDisableTiming));
            FRX_CUDA(cudaEventCreateWithFlags(&hp.computed[i], cudaEventDisableTiming));
            FRX_CUDA(cudaEventCreateWithFlags(&hp.returned[i], cudaEventDisableTiming));
        }
    }
    *pipe = &hp;
    return FRX_OK;
}
struct HostSlotBytes {
    size_t x, out, logits, gate, slot;
};
HostSlotBytes host_slot_bytes(int T, int n, int E) {
    HostSlotBytes b{};
    b.x = align_up(size_t(T) * n * 4);
    b.out = b.x;
    b.logits = align_up(size_t(T) * E * 4);
    b.gate = align_up(size_t(T) * 4);
    b.slot = b.x + b.out + b.logits + b.gate;
    return b;
}
}  // namespace

size_t frx_moe_layers_host_workspace_bytes(int T, int K, int n, int ff, int E) {
    const size_t l = frx_moe_layer_workspace_bytes(T, K, n, ff);
    if (!l || E < 1) return 0;
    return l + kHostSlots * host_slot_bytes(T, n, E).slot;
}

int frx_moe_layers_host(const void* const* experts, size_t stride, int E, const void* const* shared, int n, int ff,
                        const float* const* x_host, const float* const* logits_host, const float* const* gate_logit_host,
                        int L, int T, int K, float* const* out_host, void* ws, size_t ws_bytes, frx_stream_t stream) {
    if (!experts || !x_host || !logits_host || !out_host || !ws) return fail(FRX_ERR_ARG, "frx_moe_layers_host: null pointer");
    if (int rc = check_moe_shape("frx_moe_layers_host", n, ff, K)) return rc;
    if (L < 0 || T < 1 || E < 1) return fail(FRX_ERR_ARG, "frx_moe_layers_host: L %d, T %d, E %d", L, T, E);
    const size_t need = frx_moe_layers_host_workspace_bytes(T, K, n, ff, E);
    if (ws_bytes < need) return fail(FRX_ERR_WORKSPACE, "frx_moe_layers_host: workspace %zu < %zu", ws_bytes, need);
    for (int l = 0; l < L; ++l)
        if (!experts[l] || !x_host[l] || !logits_host[l] || !out_host[l]) return fail(FRX_ERR_ARG, "frx_moe_layers_host: null pointer for layer %d", l);
    if (L == 0) return FRX_OK;
    HostPipe* hp = nullptr;
    if (int rc = host_pipe(&hp)) return rc;
    const size_t lw = frx_moe_layer_workspace_bytes(T, K, n, ff);
    const HostSlotBytes sb = host_slot_bytes(T, n, E);
    auto* base = static_cast<uint8_t*>(ws);
    // what is already queued on the caller's stream may still use the workspace
    FRX_CUDA(cudaEventRecord(hp->start, stream));
    FRX_CUDA(cudaStreamWaitEvent(hp->in, hp->start, 0));
    for (int l = 0; l < L; ++l) {
        const int s = l % kHostSlots;
        uint8_t* slot = base + lw + size_t(s) * sb.slot;
        float* dx = reinterpret_cast<float*>(slot);
        float* dout = reinterpret_cast<float*>(slot + sb.x);
        float* dlog = reinterpret_cast<float*>(slot + sb.x + sb.out);
        float* dgate = reinterpret_cast<float*>(slot + sb.x + sb.out + sb.logits);
        const float* gh = gate_logit_host ? gate_logit_host[l] : nullptr;
        // the slot is free once the output of the layer that used it last has been copied out
        if (l >= kHostSlots) FRX_CUDA(cudaStreamWaitEvent(hp->in, hp->returned[s], 0));
        FRX_CUDA(cudaMemcpyAsync(dx, x_host[l], size_t(T) * n * 4, cudaMemcpyHostToDevice, hp->in));
        FRX_CUDA(cudaMemcpyAsync(dlog, logits_host[l], size_t(T) * E * 4, cudaMemcpyHostToDevice, hp->in));
        if (gh) FRX_CUDA(cudaMemcpyAsync(dgate, gh, size_t(T) * 4, cudaMemcpyHostToDevice, hp->in));
        FRX_CUDA(cudaEventRecord(hp->copied[s], hp->in));
        FRX_CUDA(cudaStreamWaitEvent(stream, hp->copied[s], 0));
        if (int rc = frx_moe_layer(experts[l], stride, E, shared ? shared[l] : nullptr, n, ff, dx, dlog, gh ? dgate : nullptr, T, K, dout, nullptr,
                                   nullptr, ws, lw, stream))
            return rc;
        FRX_CUDA(cudaEventRecord(hp->computed[s], stream));
        FRX_CUDA(cudaStreamWaitEvent(hp->out, hp->computed[s], 0));
        FRX_CUDA(cudaMemcpyAsync(out_host[l], dout, size_t(T) * n * 4, cudaMemcpyDeviceToHost, hp->out));
        FRX_CUDA(cudaEventRecord(hp->returned[s], hp->out));
    }
    FRX_CUDA(cudaStreamSynchronize(hp->out));
    FRX_CUDA(cudaStreamSynchronize(hp->in));
    FRX_CUDA(cudaStreamSynchronize(stream));
    return FRX_OK;
}

int frx_workspace_status(const void* ws, frx_stream_t stream) {
    if (!ws) return fail(FRX_ERR_ARG, "frx_workspace_status: null workspace");
    int st[4] = {0, 0, 0, 0};
    FRX_CUDA(cudaMemcpyAsync(st, ws, sizeof st, cudaMemcpyDeviceToHost, stream));
    FRX_CUDA(cudaStreamSynchronize(stream));
    if (st[3] != kCookie || st[0] == kDevOk) return FRX_OK;
    // reported once: the error words are cleared so that later calls on this workspace start clean
    FRX_CUDA(cudaMemsetAsync(const_cast<void*>(ws), 0, 4, stream));
    FRX_CUDA(cudaMemsetAsync(static_cast<uint8_t*>(const_cast<void*>(ws)) + 8, 0, 4, stream));
    FRX_CUDA(cudaStreamSynchronize(stream));
    switch (st[0]) {
        case kDevBadExpertId: return fail(FRX_ERR_DEVICE, "expert id out of range at slot %d", st[2]);
        case kDevWaitTimeout: return fail(FRX_ERR_DEVICE, "a kernel's bounded wait (on a shared-memory barrier or on a peer's flag) ran out");
        case kDevTooManyItems: return fail(FRX_ERR_DEVICE, "more work items than the workspace holds");
        default: return fail(FRX_ERR_DEVICE, "device error %d", st[0]);
    }
}

int frx_moe_combine(float* out, const float* yh, const float* w, const int32_t* hit_n, const float* shexp, const float* gate,
                    int n, int K, int T, frx_stream_t stream) {
    if (!out || !yh || !w) return fail(FRX_ERR_ARG, "frx_moe_combine: null pointer");
    if (n < 1 || K < 1 || T < 0) return fail(FRX_ERR_ARG, "frx_moe_combine: n %d, K %d, T %d", n, K, T);
    if (T == 0) return FRX_OK;
    FRX_LAUNCH(kKCombine, stream, k_combine_hits<<<dim3((n + 255) / 256, T), 256, 0, stream>>>(out, yh, w, hit_n, shexp, gate, n, K));
    FRX_CUDA(cudaGetLastError());
    return FRX_OK;
}

// Tuning knobs for measurements (process-wide, not thread-safe: set them before any compute call).
int frx_debug_set_down_task_weight(int sixteenths) {
    if (sixteenths < 0 || sixteenths > 64) return fail(FRX_ERR_ARG, "frx_debug_set_down_task_weight: 0 .. 64");
    g_down_heavy = sixteenths;
    return FRX_OK;
}
int frx_debug_set_down_item_weight(int sixteenths) {
    if (sixteenths < 0 || sixteenths > 4096) return fail(FRX_ERR_ARG, "frx_debug_set_down_item_weight: 0 .. 4096");
    g_down_per_item = sixteenths;
    return FRX_OK;
}
int frx_debug_set_evict_first(int on) {
    g_evict_first = on ? 1 : 0;
    return FRX_OK;
}
int frx_debug_set_fold_quant(int on) {
    g_fold_quant = on ? 1 : 0;
    return FRX_OK;
}
int frx_debug_set_stream_stamps(void* device_buffer) {
    g_stream_stamps = static_cast<unsigned long long*>(device_buffer);
    return FRX_OK;
}
int frx_debug_set_fused_ffn(int on) {
    g_fused = on ? 1 : 0;
    return FRX_OK;
}
int frx_debug_set_ffn_buffers(int gate_up, int down) {
    if (gate_up < 0 || gate_up > kMaxItemBufs4 || gate_up == 1 || down < 0 || down > kMaxItemBufs4 || down == 1)
        return fail(FRX_ERR_ARG, "frx_debug_set_ffn_buffers: 0 or 2 .. %d", kMaxItemBufs4);
    g_ffn_nbuf_g = gate_up;
    g_ffn_nbuf_d = down;
    return FRX_OK;
}
int frx_debug_set_four_group_tasks(int on) {
    g_task4 = on & 3;
    return FRX_OK;
}
int frx_debug_set_gate_up_chunks(int chunks) {
    if (chunks < 0 || chunks > 16) return FRX_ERR_ARG;
    g_gu_chunks = chunks;
    return FRX_OK;
}
int frx_debug_set_consumer_warps(int nw) {
    if (nw != 8 && nw != 12 && nw != 16 && nw != 20) return FRX_ERR_ARG;
    g_nw = nw;
    return FRX_OK;
}
int frx_debug_set_narrow_items(int on) {
    g_narrow = on ? 1 : 0;
    return FRX_OK;
}

size_t frx_moe_decode_workspace_offset(int T, int K, int n, int ff, const char* what) {
    if (!what || T < 1 || K < 1 || n < kUnitK || ff < kUnitK) return size_t(-1);
    const Layout L = make_layout(T, K, n, ff);
    const struct { const char* name; size_t off; } tab[] = {{"status", L.status}, {"items", L.items}, {"order", L.order}, {"xq", L.xq},
                                                            {"xa", L.xa}, {"xc", L.xc}, {"h", L.h}, {"hq", L.hq}, {"ha", L.ha}, {"hc", L.hc},
                                                            {"y", L.y}, {"ysh", L.ysh}};
    for (const auto& t : tab)
        if (!std::strcmp(t.name, what)) return t.off;
    return size_t(-1);
}

// ---- moe_hits
namespace {
struct HitsLayout {
    size_t status, items, xq, xa, xc, gu, h, hq, ha, hc, total;
};
HitsLayout hits_layout(int K, int n, int ff, int T) {
    HitsLayout L{};
    size_t off = 0;
    auto take = [&](size_t bytes) {
        const size_t o = off;
        off += align_up(bytes);
        return o;
    };
    L.status = take(64);
    L.items = take(size_t(T) * K * sizeof(Item));
    L.xq = take(size_t(T) * n);
    L.xa = take(size_t(T) * (n / kQ8) * 4);
    L.xc = take(size_t(T) * (n / kQ8) * 4);
    L.gu = take(size_t(T) * K * ff * 8);
    L.h = take(size_t(T) * K * ff * 4);
    L.hq = take(size_t(T) * K * ff);
    L.ha = take(size_t(T) * K * (ff / kQ8) * 4);
    L.hc = take(size_t(T) * K * (ff / kQ8) * 4);
    L.total = off;
    return L;
}
}  // namespace

size_t frx_moe_hits_scratch_bytes(int K, int n, int ff, int T) {
    if (K < 1 || T < 1 || n < kUnitK || ff < kUnitK) return 0;
    return hits_layout(K, n, ff, T).total;
}

int frx_moe_hits(const uint8_t* const* hit_ptr, const int32_t* hit_n, int K, const float* x, int n, int ff, void* scratch,
                 size_t scratch_bytes, float* yh, frx_stream_t stream, int T) {
    if (!hit_ptr || !hit_n || !x || !scratch || !yh) return fail(FRX_ERR_ARG, "frx_moe_hits: null pointer");
    if (int rc = check_moe_shape("frx_moe_hits", n, ff, K)) return rc;
    if (T < 1 || T * K > 1024) return fail(FRX_ERR_SHAPE, "frx_moe_hits: unsupported window T %d x K %d (T * K <= 1024)", T, K);
    if (uintptr_t(scratch) % kAlign || uintptr_t(x) % 16) return fail(FRX_ERR_ARG, "frx_moe_hits: scratch must be 256-byte aligned, x 16-byte aligned");
    const HitsLayout L = hits_layout(K, n, ff, T);
    if (scratch_bytes < L.total) return fail(FRX_ERR_WORKSPACE, "frx_moe_hits: scratch %zu < %zu", scratch_bytes, L.total);
    StreamCfg cfg;
    if (int rc = stream_cfg(n, ff, cfg)) return rc;
    if (int rc = set_smem_attr()) return rc;
    auto* base = static_cast<uint8_t*>(scratch);
    launch_quant_x(x, T, n, act_x(base, L), stream);
    FRX_LAUNCH(kKGroup, stream, k_group_ptr<<<1, 1024, 0, stream>>>(hit_ptr, hit_n, T, K, reinterpret_cast<Item*>(base + L.items), reinterpret_cast<int*>(base + L.status)));
    StreamParams p{};
    p.items = reinterpret_cast<const Item*>(base + L.items);
    p.status = reinterpret_cast<int*>(base + L.status);
    p.gu = reinterpret_cast<float2*>(base + L.gu);
    p.h = reinterpret_cast<float*>(base + L.h);
    p.y = yh;
    p.ysh = nullptr;
    p.n = n;
    p.ff = ff;
    p.K = K;
    p.TK = T * K;
    launch_ffn(p, act_x(base, L), act_h(base, L), size_t(T) * K, cfg, stream);
    FRX_CUDA(cudaGetLastError());
    return FRX_OK;
}

// ---- prefill-sized entry, streaming form: the general grouping feeding the same expert kernel
namespace {
struct PfLayout {
    size_t status, chunk_cnt, bounds, item_off, perm, items, xq, xa, xc, gu, h, hq, ha, hc, total;
    int n_chunks, max_items;
};
PfLayout pf_layout(int T, int K, int n, int ff, int E) {
    PfLayout L{};
    size_t off = 0;
    auto take = [&](size_t bytes) {
        const size_t o = off;
        off += align_up(bytes);
        return o;
    };
    const size_t S = size_t(T) * K;
    L.n_chunks = int((S + kChunkSlots - 1) / kChunkSlots);
    L.max_items = int(S / kTokPerItem) + E;
    L.status = take(64);
    L.chunk_cnt = take(size_t(L.n_chunks) * E * 4);
    L.bounds = take(size_t(E + 1) * 4);
    L.item_off = take(size_t(E + 1) * 4);
    L.perm = take(S * 4);
    L.items = take(size_t(L.max_items) * sizeof(Item));
    L.xq = take(size_t(T) * n);
    L.xa = take(size_t(T) * (n / kQ8) * 4);
    L.xc = take(size_t(T) * (n / kQ8) * 4);
    L.gu = take(S * ff * 8);
    L.h = take(S * ff * 4);
    L.hq = take(S * ff);
    L.ha = take(S * (ff / kQ8) * 4);
    L.hc = take(S * (ff / kQ8) * 4);
    L.total = off;
    return L;
}
// The streaming form of the prefill-sized product. With e_map (expert parallel) `experts` holds the
// E experts of this rank and slots of other experts are skipped; with xq / xd the activations
// arrive already quantized (natural order) and x is not read.
int prefill_stream_impl(const void* experts, size_t stride, int E, const int32_t* e_map, int E_all, int n, int ff, const float* x,
                        const int8_t* xq, const float* xd, const int32_t* ids, int T, int K, void* yd, void* ws, size_t ws_bytes,
                        cudaStream_t stream, int block64, int yd_bf16) {
    if (!experts || !ids || !yd || !ws) return fail(FRX_ERR_ARG, "frx_moe_prefill: null pointer");
    if (int rc = check_moe_shape("frx_moe_prefill", n, ff, K)) return rc;
    if (T < 0 || E < 1 || E > 4096 || E_all < E || E_all > 4096 || size_t(T) * K > (size_t(1) << 30))
        return fail(FRX_ERR_SHAPE, "frx_moe_prefill: unsupported T %d, E %d (of %d)", T, E, E_all);
    if ((uintptr_t(x) % 16) || (uintptr_t(xq) % 4)) return fail(FRX_ERR_ARG, "frx_moe_prefill: x must be 16-byte aligned, xq 4-byte aligned");
    if ((uintptr_t(experts) | stride) % 16 || uintptr_t(ws) % kAlign)
        return fail(FRX_ERR_ARG, "frx_moe_prefill: experts and stride must be 16-byte aligned, ws 256-byte aligned");
    if (stride < frx_q2_expert_bytes(n, ff)) return fail(FRX_ERR_ARG, "frx_moe_prefill: stride %zu < blob %zu", stride, frx_q2_expert_bytes(n, ff));
    if (T == 0) return FRX_OK;
    const PfLayout L = pf_layout(T, K, n, ff, E);
    if (ws_bytes < L.total) return fail(FRX_ERR_WORKSPACE, "frx_moe_prefill: workspace %zu < %zu", ws_bytes, L.total);
    StreamCfg cfg;
    if (int rc = stream_cfg(n, ff, cfg)) return rc;
    if (int rc = set_smem_attr()) return rc;
    auto* base = static_cast<uint8_t*>(ws);
    int* status = reinterpret_cast<int*>(base + L.status);
    int* chunk_cnt = reinterpret_cast<int*>(base + L.chunk_cnt);
    int* bounds = reinterpret_cast<int*>(base + L.bounds);
    int* item_off = reinterpret_cast<int*>(base + L.item_off);
    int32_t* perm = reinterpret_cast<int32_t*>(base + L.perm);
    Item* items = reinterpret_cast<Item*>(base + L.items);
    const int S = T * K;
    const ActBufs xb = act_x(base, L);
    if (xq) {
        const size_t nblk = size_t(T) * (n / kQ8);
        FRX_LAUNCH(kKQuant, stream, k_q8_to_frag<<<unsigned((nblk * 8 + 255) / 256), 256, 0, stream>>>(xq, xd, n, nblk, xb.q, xb.a, xb.c));
    } else {
        launch_quant_x(x, T, n, xb, stream, block64);
    }
    FRX_LAUNCH(kKGroup, stream, k_pf_hist<<<L.n_chunks, 256, size_t(E) * 4, stream>>>(ids, S, E, chunk_cnt, status, e_map, E_all));
    FRX_LAUNCH(kKGroup, stream, k_pf_scan<<<1, 1024, 0, stream>>>(chunk_cnt, L.n_chunks, E, bounds, item_off, status, L.max_items));
    FRX_LAUNCH(kKGroup, stream, k_pf_place<<<L.n_chunks, 32, size_t(E) * 4, stream>>>(ids, S, E, chunk_cnt, bounds, perm, e_map, E_all));
    FRX_LAUNCH(kKGroup, stream, k_pf_items<<<(L.max_items + 255) / 256, 256, 0, stream>>>(bounds, item_off, E, perm, static_cast<const uint8_t*>(experts), stride,
                                                             status, items));
    StreamParams p{};
    p.items = items;
    p.status = status;
    p.gu = reinterpret_cast<float2*>(base + L.gu);
    p.h = reinterpret_cast<float*>(base + L.h);
    p.y = static_cast<float*>(yd);
    p.y_bf16 = yd_bf16 ? 1 : 0;
    p.block64 = block64 ? 1 : 0;
    p.ysh = nullptr;
    p.n = n;
    p.ff = ff;
    p.K = K;
    p.TK = S;
    // the hidden-row quantizer walks the grouped slots (with an expert map: only those held here)
    // and does not keep the float hidden values, which nothing reads at these sizes
    p.row_list = perm;
    p.row_count = bounds + E;
    launch_ffn(p, xb, act_h(base, L), size_t(S), cfg, stream);
    FRX_CUDA(cudaGetLastError());
    return FRX_OK;
}

}  // namespace

size_t frx_moe_prefill_stream_workspace_bytes(int T, int K, int n, int ff, int E) {
    if (T < 1 || K < 1 || n < kUnitK || ff < kUnitK || E < 1) return 0;
    return pf_layout(T, K, n, ff, E).total;
}

int frx_moe_prefill_stream(const void* experts, size_t stride, int E, int n, int ff, const float* x, const int32_t* ids, int T, int K,
                           float* yd, void* ws, size_t ws_bytes, frx_stream_t stream) {
    return frx_moe_prefill_stream_ex(experts, stride, E, n, ff, x, ids, T, K, yd, ws, ws_bytes, stream, 0, 0);
}

int frx_moe_prefill_stream_ex(const void* experts, size_t stride, int E, int n, int ff, const float* x, const int32_t* ids, int T, int K,
                              void* yd, void* ws, size_t ws_bytes, frx_stream_t stream, int block64, int yd_bf16) {
    if (!x) return fail(FRX_ERR_ARG, "frx_moe_prefill: null pointer");
    return prefill_stream_impl(experts, stride, E, nullptr, E, n, ff, x, nullptr, nullptr, ids, T, K, yd, ws, ws_bytes, stream, block64, yd_bf16);
}

int frx_moe_prefill_stream_q8_ep(const void* experts_local, size_t stride, int E_local, const int32_t* e_map, int E_all, int n, int ff,
                                 const int8_t* xq, const float* xd, const int32_t* ids, int T, int K, float* yd, void* ws, size_t ws_bytes,
                                 frx_stream_t stream) {
    if (!xq || !xd || !e_map) return fail(FRX_ERR_ARG, "frx_moe_prefill_q8_ep: null pointer");
    return prefill_stream_impl(experts_local, stride, E_local, e_map, E_all, n, ff, nullptr, xq, xd, ids, T, K, yd, ws, ws_bytes, stream, 0, 0);
}

int frx_moe_combine_partial(float* out, const float* yd, const float* wts, const int32_t* ids, const int32_t* e_map, int n, int K, int T,
                            frx_stream_t stream) {
    if (!out || !yd || !wts || !ids || !e_map) return fail(FRX_ERR_ARG, "frx_moe_combine_partial: null pointer");
    if (n < 4 || n % 4 || K < 1 || K > 32 || T < 0) return fail(FRX_ERR_SHAPE, "frx_moe_combine_partial: n %d, K %d, T %d", n, K, T);
    if (T == 0) return FRX_OK;
    FRX_LAUNCH(kKCombine, stream, k_combine_partial<<<unsigned(T), 256, 0, stream>>>(out, yd, wts, ids, e_map, n, K));
    FRX_CUDA(cudaGetLastError());
    return FRX_OK;
}

}  // extern "C"
