// Grouping of (token, expert) slots by expert for any number of tokens: stable in slot order, no
// host synchronisation, no atomics on data, the same result on every run. Shared by the streaming
// and the tensor-memory forms of the prefill-sized entry point. Include inside namespace frx { namespace { ... } }.
#pragma once

constexpr int kCookie = 0x46525831;   // marks a workspace whose status words have been initialised

// ---------------------------------------------------------------------------------------------
// Slots are cut into chunks of 1024.
constexpr int kChunkSlots = 1024;

// Expert parallel: with `e_map` (one entry per expert of the whole layer, E_all of them), ids name
// experts of the whole layer, e_map[id] is the index of the expert among those held here or -1, and
// slots of experts held elsewhere take no part; E is then the number of experts held here.
__device__ __forceinline__ int local_expert(int id, int E, const int32_t* __restrict__ e_map, int E_all, bool& bad) {
    if (!e_map) {
        bad = id < 0 || id >= E;
        return bad ? -1 : id;
    }
    bad = id < 0 || id >= E_all;
    return bad ? -1 : e_map[id];
}

// per chunk: how many of its slots go to each expert
__global__ void __launch_bounds__(256) k_pf_hist(const int32_t* __restrict__ ids, int S, int E, int* __restrict__ chunk_cnt,
                                                 int* __restrict__ status, const int32_t* __restrict__ e_map = nullptr, int E_all = 0) {
    extern __shared__ int hist[];
    if (blockIdx.x == 0 && threadIdx.x == 0 && status[3] != kCookie) {
        status[0] = kDevOk;
        status[2] = 0;
        status[3] = kCookie;
    }
    for (int e = threadIdx.x; e < E; e += blockDim.x) hist[e] = 0;
    __syncthreads();
    const int s0 = blockIdx.x * kChunkSlots;
    for (int s = s0 + threadIdx.x; s < min(S, s0 + kChunkSlots); s += blockDim.x) {
        bool bad;
        const int e = local_expert(ids[s], E, e_map, E_all, bad);
        if (bad) {
            status[0] = kDevBadExpertId;
            status[2] = s;
        } else if (e >= 0) {
            atomicAdd(&hist[e], 1);   // integer counts: exact whatever the order
        }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) chunk_cnt[size_t(blockIdx.x) * E + e] = hist[e];
}

// per expert: exclusive offsets of its slots over the chunks (written back into chunk_cnt), its
// bounds in the grouped order, and the range of its items. bounds, item_off: [E + 1].
__global__ void __launch_bounds__(1024) k_pf_scan(int* __restrict__ chunk_cnt, int n_chunks, int E, int* __restrict__ bounds,
                                                  int* __restrict__ item_off, int* __restrict__ status, int max_items) {
    __shared__ int scan_s[1024], scan_i[1024];
    const int tid = threadIdx.x;
    const int per = (E + 1023) / 1024, e0 = tid * per, e1 = min(E, e0 + per);
    int slots = 0, items = 0;
    for (int e = e0; e < e1; ++e) {
        int run = 0;
        for (int c = 0; c < n_chunks; ++c) {
            const int v = chunk_cnt[size_t(c) * E + e];
            chunk_cnt[size_t(c) * E + e] = run;
            run += v;
        }
        bounds[e] = run;   // the count for now
        slots += run;
        items += (run + kTokPerItem - 1) / kTokPerItem;
    }
    scan_s[tid] = slots;
    scan_i[tid] = items;
    __syncthreads();
    for (int o = 1; o < 1024; o <<= 1) {
        const int a = tid >= o ? scan_s[tid - o] : 0, b = tid >= o ? scan_i[tid - o] : 0;
        __syncthreads();
        scan_s[tid] += a;
        scan_i[tid] += b;
        __syncthreads();
    }
    int at_s = scan_s[tid] - slots, at_i = scan_i[tid] - items;
    for (int e = e0; e < e1; ++e) {
        const int c = bounds[e];
        bounds[e] = at_s;
        item_off[e] = at_i;
        at_s += c;
        at_i += (c + kTokPerItem - 1) / kTokPerItem;
    }
    if (tid == 0) {
        bounds[E] = scan_s[1023];
        item_off[E] = scan_i[1023];
        if (scan_i[1023] > max_items) {
            status[0] = kDevTooManyItems;
            status[1] = 0;
        } else {
            status[1] = scan_i[1023];
        }
    }
}

// per chunk, one warp: every slot's position in the grouped order (by expert, then slot order)
__global__ void __launch_bounds__(32) k_pf_place(const int32_t* __restrict__ ids, int S, int E, const int* __restrict__ chunk_off,
                                                 const int* __restrict__ bounds, int32_t* __restrict__ perm,
                                                 const int32_t* __restrict__ e_map = nullptr, int E_all = 0) {
    extern __shared__ int cursor[];
    const int lane = threadIdx.x, c = blockIdx.x;
    for (int e = lane; e < E; e += 32) cursor[e] = bounds[e] + chunk_off[size_t(c) * E + e];
    __syncwarp();
    for (int it = 0; it < kChunkSlots / 32; ++it) {
        const int s = c * kChunkSlots + it * 32 + lane;
        bool bad = false;
        const int e = s < S ? local_expert(ids[s], E, e_map, E_all, bad) : -1;
        const bool ok = e >= 0 && e < E;
        const unsigned peers = __match_any_sync(0xffffffffu, ok ? e : -1 - lane);
        const int rank = __popc(peers & ((1u << lane) - 1));
        int pos = 0;
        if (ok) pos = cursor[e] + rank;
        __syncwarp();
        if (ok) {
            perm[pos] = s;
            if (rank == 0) cursor[e] += __popc(peers);
        }
        __syncwarp();
    }
}

