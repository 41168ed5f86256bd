// Activation quantizers of the expert path: Q8 per 32 values in the reference's natural order and in
// the fragment form the streaming kernels consume, from x, from (gate x, up x) pairs, or from codes
// that arrive already quantized. Include inside namespace frx { namespace { ... } } after frx_common.cuh.
#pragma once

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
