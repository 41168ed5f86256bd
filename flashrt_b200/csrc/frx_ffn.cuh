// Gate/up, the hidden rows and down of the decode layer as one kernel (an option, off by default).
// Include inside namespace frx { namespace { ... } } after StreamParams and frx_mma_forms.cuh.
#pragma once

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
