// Router device code: softmax over the expert logits of a token and the k most probable experts.
// Semantics of qwen4exp::moe_route_topk (arch/qwen4exp/moe_ref.cu:21-86) and of the host routing
// in moe_block (moe_ref.cu:150-170): ids in descending probability, ties to the lower index,
// weights p / max(sum of the selected p, 6.103515625e-5).
//
// One warp per token. The ranking is done on the logits themselves (softmax is monotonic, so the
// order is the same and exact ties stay exact), with one redux.sync max over an order-preserving
// integer key and one redux.sync min over the candidates' indices per selected expert. The
// probabilities are only evaluated for the softmax sum and the k winners.
#pragma once

#include "frx_common.cuh"

namespace frx {

__device__ __forceinline__ uint32_t order_key(float v) {
    const uint32_t b = __float_as_uint(v);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);   // monotonic in v; every real key > 0
}
__device__ __forceinline__ float key_value(uint32_t k) { return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k); }

// Routes token t (all 32 lanes of a warp call it). l: the token's E logits; ids_t, wts_t: its K outputs.
//
// Which logits a lane holds: when the row fills the warp exactly and is 16-byte aligned, lane L
// holds experts 128 q + 4 L .. + 3 for q = 0 .. V / 4 - 1 (V / 4 vector loads, all in flight at
// once); otherwise experts 32 i + L. Either way a lane's slots are in ascending expert order, which
// the tie rule (lowest index wins) relies on.
template <int V>   // logits per lane: E <= 32 * V
__device__ __forceinline__ void route_warp(const float* __restrict__ l, int E, int K, int lane, int32_t* __restrict__ ids_t,
                                           float* __restrict__ wts_t, uint32_t* counts, uint32_t* tail) {
    const bool vec = (V % 4 == 0) && E == 32 * V && (reinterpret_cast<uintptr_t>(l) & 15) == 0;
    auto slot_expert = [&](int i) { return vec ? 128 * (i >> 2) + 4 * lane + (i & 3) : 32 * i + lane; };
    uint32_t key[V];
    if (vec) {
        float4 v[V / 4 > 0 ? V / 4 : 1];
#pragma unroll
        for (int q = 0; q < V / 4; ++q) v[q] = reinterpret_cast<const float4*>(l)[32 * q + lane];
#pragma unroll
        for (int q = 0; q < V / 4; ++q) {   // + 0.0f: -0.0 and +0.0 tie, as they do when compared as floats
            key[4 * q] = order_key(v[q].x + 0.0f);
            key[4 * q + 1] = order_key(v[q].y + 0.0f);
            key[4 * q + 2] = order_key(v[q].z + 0.0f);
            key[4 * q + 3] = order_key(v[q].w + 0.0f);
        }
    } else {
#pragma unroll
        for (int i = 0; i < V; ++i) {
            const int e = 32 * i + lane;
            key[i] = e < E ? order_key(l[e] + 0.0f) : 0u;
        }
    }
    // every lane keeps its best and its second best key (with their experts): when its best is
    // taken, the second moves up without a rescan; the lane rescans only when it is hit again
    uint32_t best = 0, next = 0;
    int best_i = 0x7fffffff, next_i = 0x7fffffff;
    auto rescan = [&]() {
        best = 0;
        next = 0;
        best_i = 0x7fffffff;
        next_i = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < V; ++i) {
            const uint32_t kv = key[i];
            if (kv > best) {   // ascending index within a lane: the first maximum wins
                next = best;
                next_i = best_i;
                best = kv;
                best_i = slot_expert(i);
            } else if (kv > next) {
                next = kv;
                next_i = slot_expert(i);
            }
        }
    };
    rescan();
    bool next_valid = true;
    const uint32_t kmax = __reduce_max_sync(0xffffffffu, best);
    const float m = key_value(kmax);
    double part[4] = {0.0, 0.0, 0.0, 0.0};   // four running sums: the additions are slow and would otherwise form one chain
#pragma unroll
    for (int i = 0; i < V; ++i)
        if (key[i] != 0u) part[i & 3] += double(expf(key_value(key[i]) - m));
    double sum = (part[0] + part[1]) + (part[2] + part[3]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);

    // selection: K rounds on the integer keys only; lane k remembers the k-th winner
    uint32_t my_key = 0;
    int my_id = 0;
    for (int k = 0; k < K; ++k) {
        const uint32_t top = __reduce_max_sync(0xffffffffu, best);
        const int sel = __reduce_min_sync(0xffffffffu, best == top ? best_i : 0x7fffffff);
        if ((vec ? (sel >> 2) & 31 : sel & 31) == lane) {   // the owner retires it and moves its next best up
#pragma unroll
            for (int i = 0; i < V; ++i)
                if (slot_expert(i) == sel) key[i] = 0u;
            if (next_valid) {
                best = next;
                best_i = next_i;
                next_valid = false;
            } else {
                rescan();
                next_valid = true;
            }
        }
        if (lane == k) {
            my_key = top;
            my_id = sel;
        }
    }
    // probabilities of the winners, all lanes at once; their sum in selection order (lane order)
    const float my_p = lane < K ? float(double(expf(key_value(my_key) - m)) / sum) : 0.0f;
    float wsum = 0.0f;
    for (int k = 0; k < K; ++k) wsum += __shfl_sync(0xffffffffu, my_p, k);
    wsum = fmaxf(wsum, 6.103515625e-5f);
    if (lane < K) {
        ids_t[lane] = my_id;
        wts_t[lane] = __fdiv_rn(my_p, wsum);
        if (counts) atomicAdd(counts + my_id, 1u);
        if (tail) atomicAdd(tail + my_id, 1u);
    }
}


}  // namespace frx
