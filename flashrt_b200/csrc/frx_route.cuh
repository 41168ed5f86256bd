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
template <int V>   // logits per lane: E <= 32 * V
__device__ __forceinline__ void route_warp(const float* __restrict__ l, int E, int K, int lane, int32_t* __restrict__ ids_t,
                                           float* __restrict__ wts_t, uint32_t* counts, uint32_t* tail) {
    uint32_t key[V];
    uint32_t best = 0;
    int best_i = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < V; ++i) {
        const int e = 32 * i + lane;
        key[i] = e < E ? order_key(l[e] + 0.0f) : 0u;   // + 0.0f: -0.0 and +0.0 tie, as they do when compared as floats
        if (key[i] > best) {   // ascending index within a lane: the first maximum wins
            best = key[i];
            best_i = e;
        }
    }
    const uint32_t kmax = __reduce_max_sync(0xffffffffu, best);
    const float m = key_value(kmax);
    double part = 0.0;
#pragma unroll
    for (int i = 0; i < V; ++i)
        if (32 * i + lane < E) part += double(expf(key_value(key[i]) - m));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
    const double sum = part;

    // selection: K rounds on the integer keys only; lane k remembers the k-th winner
    uint32_t my_key = 0;
    int my_id = 0;
    for (int k = 0; k < K; ++k) {
        const uint32_t top = __reduce_max_sync(0xffffffffu, best);
        const int sel = __reduce_min_sync(0xffffffffu, best == top ? best_i : 0x7fffffff);
        if ((sel & 31) == lane) {   // the owner retires it and finds its next best
            best = 0;
            best_i = 0x7fffffff;
#pragma unroll
            for (int i = 0; i < V; ++i) {
                if (32 * i + lane == sel) key[i] = 0u;
                if (key[i] > best) {
                    best = key[i];
                    best_i = 32 * i + lane;
                }
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
