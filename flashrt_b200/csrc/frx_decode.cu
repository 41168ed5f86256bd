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

#include "frx_quant.cuh"

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

#include "frx_mma_forms.cuh"

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

#include "frx_ffn.cuh"

#include "frx_combine.cuh"

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
int g_small4 = 0, g_small8 = 8;   // launches of at most this many tasks per SM take blocks of 4 / 8 warps with deeper rings (measured at 1 to 3 tokens: 8 warps 26.9 us per layer, 4 warps 27.7, 16 warps 28.9)
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
        if (max_tasks > 0 && max_tasks <= (long long)g_small4 * sms) first = 4;
        else if (max_tasks > 0 && max_tasks <= (long long)g_small8 * sms) first = 8;
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
int frx_debug_set_small_launch_limits(int four_warps, int eight_warps) {
    if (four_warps < 0 || eight_warps < four_warps) return FRX_ERR_ARG;
    g_small4 = four_warps;
    g_small8 = eight_warps;
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
