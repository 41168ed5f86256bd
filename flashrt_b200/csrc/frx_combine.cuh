// The combine kernels of the expert path: the ordered weighted sum of a token's expert outputs plus
// the shared expert, the same with the expert-parallel all-reduce over peer memory inside, the
// partial sum of the experts one rank holds, and moe_hits' combine. Include inside
// namespace frx { namespace { ... } } after frx_common.cuh.
#pragma once

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
