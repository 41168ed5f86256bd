// Prefill-sized grouped expert product (moe_q2::run, kernels/cuda/moe_q2.h:21-30) on the
// 5th-generation tensor cores: tcgen05.mma with fp32 accumulators in tensor memory.
//
// Numerics are the decode path's, i.e. the reference CPU path's: int8 activation codes per 32
// values, exact integer dot products per 32-block, then scale and accumulate in the reference's
// order and roundings. The tensor core does only the exact part. Operands are small integers held
// in fp16 -- the weight codes q - 1 in {-1, 0, 1, 2} and the activation codes in [-127, 127] -- so
// every product and every partial sum of one 32-block (|sum| <= 8128) is exact in the fp32
// accumulator. Each 64-weight block therefore yields two accumulators S0, S1 per (row, token) in
// tensor memory, which the epilogue warps turn into d * (a0 * S0 + a1 * S1) and add to running
// sums held in registers, block after block.
//
// Per CTA (one per SM), warp roles: 0 = TMA producer, 1 = MMA issuer and tensor-memory owner,
// 2-3 = dequant (2-bit codes of 128 rows x 64 weights -> fp16 core-matrix layout in shared
// memory), 4-19 = epilogue (tensor memory -> registers, scaling, stores of the (gate, up) sums or
// the output rows): each epilogue warp owns 32 rows (its quarter of the tensor-memory lanes) x 32
// token columns. 640 threads leave 96 registers per thread, which lets an epilogue thread fetch
// 16 columns of both sums per round trip to tensor memory (a round trip costs several hundred
// cycles whatever its size). Hand-offs are shared-memory barriers; a barrier operation has about a
// hundred cycles of latency and a thread's steps are serial, so each role tests the next step's
// barriers while it still works on the current one.
// All waits are bounded; a wait that runs out sets the workspace status word and the block drains.
#include "frx_umma.cuh"

#include <cuda_bf16.h>

#include <mutex>

namespace frx {
namespace {

#include "frx_group.cuh"

constexpr int kTileRows = 128;     // M of the MMA: 8 groups of 16 matrix rows
constexpr int kTileTok = 128;      // most tokens of one tile (N of the MMA), a multiple of 16
constexpr int kTokPad = 16;        // every expert's token count is padded to this
// fp16 A tile of one 64-block: 16 groups of 8 rows, each 8 core matrices (8 rows x 16 bytes) 192
// bytes apart rather than 128, so that the dequant warps' 8-byte stores to two neighbouring
// chunks fall into different banks
constexpr int kALbo = 192, kASbo = 8 * kALbo;
constexpr int kStepBytesA = (kTileRows / 8) * kASbo;   // 24 KB
constexpr int kStepBytesB = kTileTok * 64 * 2;    // fp16 B tile of one 64-block: 16 KB
constexpr int kStepBytesS = kTileTok * 8;         // activation scales of one 64-block: 1 KB
constexpr int kUnitTileBytes = 8 * kUnitBytes;    // packed weights of 8 groups x one unit: 4608 B
constexpr int kStagesW = 8, kStagesA = 4, kStagesB = 4, kStagesD = 2;
static_assert(kStagesA == kStagesB, "one barrier frees an A and a B stage together");
constexpr int kStageColsD = 2 * kTileTok;   // tensor-memory columns of one step: the two 32-value sums of every token
static_assert(kStagesD * kStageColsD <= 512, "tensor memory has 512 columns");
constexpr int kWarpsDequant = 2, kWarpsEpilogue = 16;
constexpr int kThreads = (2 + kWarpsDequant + kWarpsEpilogue) * 32;   // 640: 96 registers per thread
constexpr int kGroupsPerDequantWarp = 8 / kWarpsDequant;             // 16-row groups of the tile per dequant warp

// meta words: [0] padded positions in use, [1] token blocks
struct PfuLayout {
    size_t status, chunk_cnt, bounds, item_off, perm, pb, tbo, meta, tb_e, tb_p0, tb_n, pslot, xq, xd, xg, xa, hf, hg, ha, total;
    int n_chunks, max_tb;
    size_t pmax;
};

PfuLayout pfu_layout(int T, int K, int n, int ff, int E) {
    PfuLayout L{};
    size_t off = 0;
    auto take = [&](size_t bytes) {
        const size_t o = off;
        off += align_up(bytes);
        return o;
    };
    const size_t S = size_t(T) * K;
    L.n_chunks = int((S + kChunkSlots - 1) / kChunkSlots);
    L.pmax = align_up(S + size_t(kTokPad) * size_t(E < int(S) ? E : int(S)), 128);
    L.max_tb = int(S / kTileTok) + E + 1;
    L.status = take(64);
    L.chunk_cnt = take(size_t(L.n_chunks) * E * 4);
    L.bounds = take(size_t(E + 1) * 4);
    L.item_off = take(size_t(E + 1) * 4);
    L.perm = take(S * 4);
    L.pb = take(size_t(E + 1) * 4);
    L.tbo = take(size_t(E + 1) * 4);
    L.meta = take(64);
    L.tb_e = take(size_t(L.max_tb) * 4);
    L.tb_p0 = take(size_t(L.max_tb) * 4);
    L.tb_n = take(size_t(L.max_tb) * 4);
    L.pslot = take(L.pmax * 4);
    L.xq = take(size_t(T) * n);
    L.xd = take(size_t(T) * (n / kQ8) * 4);
    L.xg = take(L.pmax * n * 2);
    L.xa = take(L.pmax * (n / kQK) * 8);
    L.hf = take(L.pmax * ff * 8);   // (gate x, up x) pairs
    L.hg = take(L.pmax * ff * 2);
    L.ha = take(L.pmax * (ff / kQK) * 8);
    L.total = off;
    return L;
}

// ---------------------------------------------------------------------------------------------
// Plan: pad every expert's slot count to 16 (padded position space p), cut it into token blocks of
// at most 128. One block of 1024 threads.
__global__ void __launch_bounds__(1024) k_pfu_plan(const int* __restrict__ bounds, int E, int* __restrict__ pb, int* __restrict__ tbo,
                                                   int* __restrict__ meta, int* __restrict__ tb_e, int* __restrict__ tb_p0,
                                                   int* __restrict__ tb_n, int max_tb, int* __restrict__ status) {
    __shared__ int scan_p[1024], scan_t[1024];
    const int tid = threadIdx.x;
    const int per = (E + 1023) / 1024, e0 = tid * per, e1 = min(E, e0 + per);
    int pp = 0, tt = 0;
    for (int e = e0; e < e1; ++e) {
        const int c = bounds[e + 1] - bounds[e];
        pp += (c + kTokPad - 1) / kTokPad * kTokPad;
        tt += (c + kTileTok - 1) / kTileTok;
    }
    scan_p[tid] = pp;
    scan_t[tid] = tt;
    __syncthreads();
    for (int o = 1; o < 1024; o <<= 1) {
        const int a = tid >= o ? scan_p[tid - o] : 0, b = tid >= o ? scan_t[tid - o] : 0;
        __syncthreads();
        scan_p[tid] += a;
        scan_t[tid] += b;
        __syncthreads();
    }
    const int n_tb = scan_t[1023];
    if (n_tb > max_tb) {
        if (tid == 0) {
            status[0] = kDevTooManyItems;
            meta[0] = 0;
            meta[1] = 0;
        }
        return;
    }
    int at_p = scan_p[tid] - pp, at_t = scan_t[tid] - tt;
    for (int e = e0; e < e1; ++e) {
        const int c = bounds[e + 1] - bounds[e], pc = (c + kTokPad - 1) / kTokPad * kTokPad;
        pb[e] = at_p;
        tbo[e] = at_t;
        for (int j = 0; j * kTileTok < c; ++j) {
            tb_e[at_t] = e;
            tb_p0[at_t] = at_p + j * kTileTok;
            tb_n[at_t] = min(kTileTok, pc - j * kTileTok);
            ++at_t;
        }
        at_p += pc;
    }
    if (tid == 0) {
        pb[E] = scan_p[1023];
        tbo[E] = n_tb;
        meta[0] = scan_p[1023];
        meta[1] = n_tb;
    }
}

// Offset, in bytes, of the 16-byte chunk `c` (8 fp16 values of K) of padded position p in the
// grouped fp16 operand: [64-block][p / 8][chunk 0..7][p % 8][16 bytes] -- the MMA's K-major
// core-matrix order, so a token block's tile for one 64-block is one contiguous range.
__device__ __forceinline__ size_t grouped_chunk_off(size_t pmax, int b64, int p, int chunk) {
    return (((size_t(b64) * (pmax / 8) + size_t(p >> 3)) * 8 + size_t(chunk)) * 8 + size_t(p & 7)) * 16;
}
// Activation scales: [64-block][p / 2][a0 of p even, a0 of p odd, a1 of p even, a1 of p odd].
__device__ __forceinline__ size_t grouped_scale_idx(size_t pmax, int b64, int p, int half) {
    return (size_t(b64) * pmax + size_t(p & ~1)) * 2 + size_t(half) * 2 + size_t(p & 1);
}

// Gather: for every padded position, its slot (or -1), the int8 codes of the slot's token as fp16
// in the grouped operand layout, and the token's block scales. Block = 8 positions x 32 chunks.
__global__ void __launch_bounds__(256) k_pfu_gather(const int* __restrict__ bounds, const int* __restrict__ pb, int E,
                                                    const int32_t* __restrict__ perm, const int* __restrict__ meta, int K, int n,
                                                    size_t pmax, const int8_t* __restrict__ xq, const float* __restrict__ xd,
                                                    uint8_t* __restrict__ xg, float* __restrict__ xa, int32_t* __restrict__ pslot) {
    const int r = threadIdx.x & 7, cl = threadIdx.x >> 3;
    const int p = blockIdx.x * 8 + r;
    if (blockIdx.x * 8 >= meta[0]) return;
    int lo = 0, hi = E;   // the expert whose padded range holds p
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (pb[mid] <= p) lo = mid; else hi = mid;
    }
    const int e = lo, k = p - pb[e], c = bounds[e + 1] - bounds[e];
    const int slot = (p < meta[0] && k < c) ? perm[bounds[e] + k] : -1;
    if (cl == 0) pslot[p] = slot;
    const int t = slot >= 0 ? slot / K : 0;
    const int chunks = n / 8, nb = n / kQK;
    for (int ch = cl; ch < chunks; ch += 32) {
        uint4 out = make_uint4(0u, 0u, 0u, 0u);
        if (slot >= 0) {
            const uint2 q = *reinterpret_cast<const uint2*>(xq + size_t(t) * n + size_t(ch) * 8);
            const int8_t* b = reinterpret_cast<const int8_t*>(&q);
            __half2 h[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) h[i] = __halves2half2(__int2half_rn(int(b[2 * i])), __int2half_rn(int(b[2 * i + 1])));
            out = *reinterpret_cast<const uint4*>(h);
        }
        *reinterpret_cast<uint4*>(xg + grouped_chunk_off(pmax, ch >> 3, p, ch & 7)) = out;
    }
    for (int b = cl; b < nb; b += 32) {
        const float a0 = slot >= 0 ? xd[size_t(t) * (n / kQ8) + 2 * b] : 0.0f;
        const float a1 = slot >= 0 ? xd[size_t(t) * (n / kQ8) + 2 * b + 1] : 0.0f;
        xa[grouped_scale_idx(pmax, b, p, 0)] = a0;
        xa[grouped_scale_idx(pmax, b, p, 1)] = a1;
    }
}

// Natural-order Q8 of x rows (q2_0::quantize_q8): warp per 32-block.
__device__ __forceinline__ int q8_block_pf(float v, float& d_out, float partner) {
    float am = fmaxf(fabsf(v), fabsf(partner));   // partner: the other half of a 64-value scale block (block64), else 0
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
    const float d = __fdiv_rn(am, 127.0f);
    const float id = d != 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
    d_out = __half2float(__float2half_rn(d));
    return int(round_half_away(__fmul_rn(v, id)));
}

__global__ void __launch_bounds__(256) k_pfu_quant_x(const float* __restrict__ x, size_t n_blocks, int8_t* __restrict__ q,
                                                     float* __restrict__ d, int block64) {
    const size_t blk = size_t(blockIdx.x) * 8 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (blk >= n_blocks) return;
    float dd;
    const int c = q8_block_pf(x[blk * kQ8 + lane], dd, block64 ? x[(blk ^ 1) * kQ8 + lane] : 0.0f);
    q[blk * kQ8 + lane] = int8_t(c);
    if (lane == 0) d[blk] = dd;
}

// Q8 of the hidden rows (one row of ff per padded position) straight into the grouped fp16
// operand layout and scale table of the down product. A thread owns 8 consecutive hidden values
// (one 16-byte chunk of the operand), four neighbouring lanes one 32-block: silu(gate x) * up x is
// formed here (eight independent exponentials per thread hide their latency), the block maximum
// comes from two shuffles, and each thread stores its chunk whole.
__global__ void __launch_bounds__(256) k_pfu_quant_h(const float2* __restrict__ hf, int ff, size_t pmax, const int* __restrict__ meta,
                                                     const int32_t* __restrict__ pslot, uint8_t* __restrict__ hg, float* __restrict__ ha,
                                                     int block64) {
    const int cpr = ff / 8;   // chunks per row
    const size_t chunk = size_t(blockIdx.x) * 256 + threadIdx.x;
    const size_t p = chunk / cpr;
    const bool in_range = p < size_t(meta[0]);   // no early exit: the shuffles below need the whole warp
    const int c = int(chunk % cpr);              // chunk of the row: values 8 c .. 8 c + 7
    const bool live = in_range && pslot[p] >= 0;
    float hv[8];
    float am = 0.0f;
    if (live) {
        const float4* src = reinterpret_cast<const float4*>(hf + p * ff + size_t(c) * 8);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float4 gu = src[i];   // (gate, up) of two hidden values
            hv[2 * i] = swiglu_ref(gu.x, gu.y);
            hv[2 * i + 1] = swiglu_ref(gu.z, gu.w);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) am = fmaxf(am, fabsf(hv[i]));
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) hv[i] = 0.0f;
    }
    am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 1));
    am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 2));
    if (block64) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 4));   // eight lanes hold one 64-value scale block
    // quant/q2_0/q2_0.cpp:101-113: d = amax / 127, id = 1 / d, q = roundf(v * id), d through fp16
    const float d = __fdiv_rn(am, 127.0f);
    const float id = d != 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
    __half2 h[4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
        h[i] = __halves2half2(__int2half_rn(int(round_half_away(__fmul_rn(hv[2 * i], id)))),
                              __int2half_rn(int(round_half_away(__fmul_rn(hv[2 * i + 1], id)))));
    const int b64 = c >> 3, k8 = c & 7;   // the 64-block and the chunk inside it
    if (!in_range) return;
    *reinterpret_cast<uint4*>(hg + grouped_chunk_off(pmax, b64, int(p), k8)) = *reinterpret_cast<const uint4*>(h);
    if ((c & 3) == 0) ha[grouped_scale_idx(pmax, b64, int(p), k8 >> 2)] = __half2float(__float2half_rn(d));
}

// ---------------------------------------------------------------------------------------------
struct UmmaParams {
    const uint8_t* experts;   // tiled blobs
    size_t stride;
    const int* meta;          // [1] = token blocks
    const int* tb_e;
    const int* tb_p0;
    const int* tb_n;
    const uint8_t* act;       // grouped fp16 codes (xg or hg)
    const float* act_scale;   // grouped block scales (xa or ha)
    const int32_t* pslot;
    float2* hf;               // gate/up: (gate x, up x) of every hidden element [pmax][ff]
    float* yd;                // down: [slots][n]
    int* status;
    size_t pmax;
    unsigned long long wait_ns;   // the longest a wait on a shared-memory barrier may last
    int n, ff;
    int y_bf16;               // down: yd holds bf16 rows
};

struct PfSmem {
    uint32_t w, a, b, s, sw, bars, tmem, abort, total;
};
__host__ __device__ constexpr PfSmem pf_smem() {
    PfSmem m{};
    uint32_t off = 0;
    m.w = off;
    off += kStagesW * kUnitTileBytes;
    off = (off + 1023u) & ~1023u;
    m.a = off;
    off += kStagesA * kStepBytesA;
    m.b = off;
    off += kStagesB * kStepBytesB;
    m.s = off;
    off += kStagesB * kStepBytesS;
    m.sw = off;
    off += kStagesA * kTileRows * 4;
    m.bars = off;
    off += 48 * 8;
    m.tmem = off;
    off += 16;
    m.abort = off;
    off += 16;
    m.total = off;
    return m;
}

// Barrier indices
enum : int {
    kBarWFull = 0,                      // + stage: packed weights of a unit have landed
    kBarWFree = kBarWFull + kStagesW,   // dequant warps are done with them
    kBarAFull = kBarWFree + kStagesW,   // fp16 A tile written
    kBarAFree = kBarAFull + kStagesA,   // the epilogue is done with a step's row and activation scales (and so the MMAs that
                                        // read its A and B tiles have completed): frees the A stage and the B stage of the step
    kBarBFull = kBarAFree + kStagesA,   // fp16 B tile and activation scales have landed
    kBarDFull = kBarBFull + kStagesB,   // accumulators of a step are complete in tensor memory
    kBarDFree = kBarDFull + kStagesD,   // epilogue warps have read them
    kBarCount = kBarDFree + kStagesD
};
static_assert(kBarCount <= 48, "barrier block too small");

// 8 fp32 columns of tensor memory for this thread's lane, packed in pairs.
__device__ __forceinline__ void tmem_ld8_pairs(uint32_t taddr, uint64_t (&v)[4]) {
    asm volatile(
        "{\n\t.reg .b32 r<8>;\n\t"
        "tcgen05.ld.sync.aligned.32x32b.x8.b32 {r0,r1,r2,r3,r4,r5,r6,r7}, [%4];\n\t"
        "mov.b64 %0, {r0,r1};\n\tmov.b64 %1, {r2,r3};\n\tmov.b64 %2, {r4,r5};\n\tmov.b64 %3, {r6,r7};\n\t}"
        : "=l"(v[0]), "=l"(v[1]), "=l"(v[2]), "=l"(v[3])
        : "r"(taddr));
}

template <bool GATE_UP>
__global__ void __launch_bounds__(kThreads, 1) k_pf_umma(const UmmaParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    constexpr PfSmem sm = pf_smem();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + sm.bars);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + sm.tmem);
    volatile int* abort = reinterpret_cast<volatile int*>(smem + sm.abort);

    const int kdim = GATE_UP ? p.n : p.ff;
    const int steps = kdim / kQK;                       // 64-blocks of K
    const int row_blocks = GATE_UP ? (2 * p.ff) / kTileRows : p.n / kTileRows;
    const uint32_t group_bytes = uint32_t(kdim / kUnitK) * kUnitBytes;
    const size_t section = GATE_UP ? 0 : size_t(p.ff / 8) * (size_t(p.n / kUnitK) * kUnitBytes);
    const int n_tiles = p.meta[1] * row_blocks;

    if (threadIdx.x == 0) {
        for (int i = 0; i < kStagesW; ++i) {
            mbar_init(bars + kBarWFull + i, 1);
            mbar_init(bars + kBarWFree + i, kWarpsDequant);
        }
        for (int i = 0; i < kStagesA; ++i) {
            mbar_init(bars + kBarAFull + i, kWarpsDequant);
            mbar_init(bars + kBarAFree + i, kWarpsEpilogue);
        }
        for (int i = 0; i < kStagesB; ++i) {
            mbar_init(bars + kBarBFull + i, 1);
        }
        for (int i = 0; i < kStagesD; ++i) {
            mbar_init(bars + kBarDFull + i, 1);
            mbar_init(bars + kBarDFree + i, kWarpsEpilogue);
        }
        *abort = 0;
        mbar_fence_init();
    }
    if (warp == 1) tmem_alloc(tmem_slot, 512);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;

    // "free" barriers are waited on with the parity of the phase before the one about to be used,
    // which a fresh barrier reports as complete
    auto wait_full = [&](int bar, uint32_t use) { return mbar_wait_bounded<false>(bars + bar, use & 1u, abort, p.wait_ns); };
    auto wait_free = [&](int bar, uint32_t use) { return mbar_wait_bounded<false>(bars + bar, (use & 1u) ^ 1u, abort, p.wait_ns); };

    if (warp == 0) {
        // ---------------- producer
        if (lane == 0) {
            uint32_t g = 0, gu = 0;   // steps and units issued so far
            for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
                const int tb = tile / row_blocks, rb = tile % row_blocks;
                const int e = p.tb_e[tb], p0 = p.tb_p0[tb], ntok = p.tb_n[tb];
                const uint8_t* wsrc = p.experts + size_t(e) * p.stride + section + size_t(rb) * 8 * group_bytes;
                for (int b = 0; b < steps; ++b, ++g) {
                    if ((b & 1) == 0) {
                        const uint32_t ws = gu % kStagesW;
                        wait_free(kBarWFree + ws, gu / kStagesW);
                        mbar_expect_tx(bars + kBarWFull + ws, kUnitTileBytes);
                        for (int gi = 0; gi < 8; ++gi)
                            bulk_g2s(smem + sm.w + ws * kUnitTileBytes + gi * kUnitBytes, wsrc + size_t(gi) * group_bytes + size_t(b >> 1) * kUnitBytes,
                                     kUnitBytes, bars + kBarWFull + ws);
                        ++gu;
                    }
                    const uint32_t bs = g % kStagesB;
                    wait_free(kBarAFree + bs, g / kStagesB);
                    const uint32_t bbytes = uint32_t(ntok) * 128u, sbytes = uint32_t(ntok) * 8u;
                    mbar_expect_tx(bars + kBarBFull + bs, bbytes + sbytes);
                    bulk_g2s(smem + sm.b + bs * kStepBytesB, p.act + (size_t(b) * (p.pmax / 8) + size_t(p0 >> 3)) * 1024, bbytes, bars + kBarBFull + bs);
                    bulk_g2s(smem + sm.s + bs * kStepBytesS, p.act_scale + (size_t(b) * p.pmax + size_t(p0)) * 2, sbytes, bars + kBarBFull + bs);
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer
        if (lane == 0) {
            uint32_t g = 0;
            bool a_ok = false, b_ok = false, d_ok = false;
            for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
                const int ntok = p.tb_n[tile / row_blocks];
                const uint32_t idesc = umma_idesc_f16(kTileRows, ntok);
                for (int b = 0; b < steps; ++b, ++g) {
                    const uint32_t as = g % kStagesA, bs = g % kStagesB, ds = g % kStagesD;
                    if (!a_ok) wait_full(kBarAFull + as, g / kStagesA);
                    if (!b_ok) wait_full(kBarBFull + bs, g / kStagesB);
                    if (!d_ok) wait_free(kBarDFree + ds, g / kStagesD);
                    // the next step's tests, answered while this step's MMAs are being issued
                    a_ok = mbar_try_wait(bars + kBarAFull + (g + 1) % kStagesA, ((g + 1) / kStagesA) & 1u);
                    b_ok = mbar_try_wait(bars + kBarBFull + (g + 1) % kStagesB, ((g + 1) / kStagesB) & 1u);
                    d_ok = mbar_try_wait(bars + kBarDFree + (g + 1) % kStagesD, (((g + 1) / kStagesD) & 1u) ^ 1u);
                    tc_fence_after_sync();
                    const uint32_t a_addr = smem_u32(smem + sm.a + as * kStepBytesA), b_addr = smem_u32(smem + sm.b + bs * kStepBytesB);
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk) {   // four K = 16 instructions: two per 32-block
                        const uint64_t da = umma_desc(a_addr + kk * 2 * kALbo, kALbo, kASbo), db = umma_desc(b_addr + kk * 256, 128, 1024);
                        umma_f16(tmem + ds * kStageColsD + (kk >> 1) * kTileTok, da, db, idesc, kk & 1);
                    }
                    // one commit per step: the epilogue warps release the A and B stages after they
                    // have seen it, which also tells that the MMAs are done reading those stages
                    umma_commit(bars + kBarDFull + ds);
                }
            }
        }
    } else if (warp < 2 + kWarpsDequant) {
        // ---------------- dequant: packed 2-bit codes -> fp16 (q - 1) in the A tile
        const int dw = warp - 2;   // the group (16 rows) of the tile this warp unpacks
        const int g8 = lane >> 2, t4 = lane & 3;
        const __half2 k1025 = __floats2half2_rn(1025.0f, 1025.0f);
        uint32_t g = 0, gu = 0;
        bool a_free = false, w_ready = false;   // the next step's A stage / weights were already seen free / landed
        for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
            for (int b = 0; b < steps; ++b, ++g) {
                const int j = b & 1;
                const uint32_t ws = gu % kStagesW, as = g % kStagesA;
                // (the tests were issued during the previous step's work, see the epilogue)
                if (j == 0 && !w_ready) wait_full(kBarWFull + ws, gu / kStagesW);
                // an A stage (the fp16 tile and its row scales) is free once the MMAs that read the
                // tile have completed and the epilogue warps have used the scales
                if (!a_free) wait_free(kBarAFree + as, g / kStagesA);
                uint8_t* at = smem + sm.a + as * kStepBytesA;
                uint4 wvs[kGroupsPerDequantWarp];
#pragma unroll
                for (int gi = 0; gi < kGroupsPerDequantWarp; ++gi)   // words [h][j] of this lane, per group
                    wvs[gi] = *reinterpret_cast<const uint4*>(smem + sm.w + ws * kUnitTileBytes + (dw * kGroupsPerDequantWarp + gi) * kUnitBytes + lane * 16);
                a_free = mbar_try_wait(bars + kBarAFree + (g + 1) % kStagesA, (((g + 1) / kStagesA) & 1u) ^ 1u);
                if (j == 1) w_ready = mbar_try_wait(bars + kBarWFull + (gu + 1) % kStagesW, ((gu + 1) / kStagesW) & 1u);
#pragma unroll
                for (int gh = 0; gh < 2 * kGroupsPerDequantWarp; ++gh) {
                    const int gi = gh >> 1, h = gh & 1;
                    const uint4 wv = wvs[gi];
                    const uint32_t w = h ? (j ? wv.w : wv.z) : (j ? wv.y : wv.x);
                    const int row = (dw * kGroupsPerDequantWarp + gi) * 16 + g8 + 8 * h;
                    uint8_t* dst = at + (row >> 3) * kASbo + (row & 7) * 16 + (t4 & 1) * 8;
#pragma unroll
                    for (int f = 0; f < 4; ++f) {   // field f: elements 16 f + 4 t4 .. + 3 of the block
                        const uint32_t x = (w >> (2 * f)) & 0x03030303u;
                        uint32_t lo = __byte_perm(x, 0x64646464u, 0x5140), hi = __byte_perm(x, 0x64646464u, 0x7362);   // fp16 1024 + q
                        const __half2 l2 = __hsub2(*reinterpret_cast<__half2*>(&lo), k1025), h2 = __hsub2(*reinterpret_cast<__half2*>(&hi), k1025);
                        uint2 out;
                        out.x = *reinterpret_cast<const uint32_t*>(&l2);
                        out.y = *reinterpret_cast<const uint32_t*>(&h2);
                        *reinterpret_cast<uint2*>(dst + (2 * f + (t4 >> 1)) * kALbo) = out;
                    }
                }
#pragma unroll
                for (int r = lane; r < 16 * kGroupsPerDequantWarp; r += 32) {   // this step's weight scales of the warp's rows
                    const int gi = r >> 4, l16 = r & 15;
                    const uint8_t* wt = smem + sm.w + ws * kUnitTileBytes + (dw * kGroupsPerDequantWarp + gi) * kUnitBytes;
                    const __half sc = *reinterpret_cast<const __half*>(wt + kUnitCodeBytes + (l16 & 7) * 8 + ((l16 >> 3) * 2 + j) * 2);
                    reinterpret_cast<float*>(smem + sm.sw)[as * kTileRows + (dw * kGroupsPerDequantWarp + gi) * 16 + l16] = __half2float(sc);
                }
                fence_async_smem();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(bars + kBarAFull + as);
                    if (j == 1) mbar_arrive(bars + kBarWFree + ws);
                }
                if (j == 1) ++gu;
            }
        }
    } else {
        // ---------------- epilogue
        const int ew = warp - (2 + kWarpsDequant);
        const int quarter = warp & 3;             // the tensor-memory lanes this warp may read
        const int cq = ew >> 2;                   // which 32 token columns
        const int row = quarter * 32 + lane;      // M row of the tile
        const uint32_t lane_addr = uint32_t(quarter * 32) << 16;
        uint32_t g = 0;
        bool d_ready = false;   // this step's accumulators were already seen complete
        for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
            const int tb = tile / row_blocks, rb = tile % row_blocks;
            const int p0 = p.tb_p0[tb], ntok = p.tb_n[tb];
            const int ncols = max(0, min(32, ntok - 32 * cq));
            const int last_chunk = ncols > 0 ? (ncols - 1) >> 4 : 0;   // the last 16-column chunk this thread reads
            float acc[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) acc[i] = 0.0f;
            for (int b = 0; b < steps; ++b, ++g) {
                const uint32_t as = g % kStagesA, bs = g % kStagesB, ds = g % kStagesD;
                // Every barrier operation costs on the order of a hundred cycles of latency, and a
                // thread's steps are serial (its sums are added block after block), so the tests
                // are issued ahead of where their answer is needed: the one for this step's
                // accumulators was issued during the previous step's arithmetic.
                if (!d_ready) wait_full(kBarDFull + ds, g / kStagesD);
                tc_fence_after_sync();
                // complete long ago (the MMAs needed them); tested so that what the dequant warps
                // (row scales) and the TMA (activation scales) wrote is acquired by this thread
                bool a_ready = mbar_try_wait(bars + kBarAFull + as, (g / kStagesA) & 1u);
                bool b_ready = mbar_try_wait(bars + kBarBFull + bs, (g / kStagesB) & 1u);
                const uint32_t t0 = tmem + lane_addr + ds * kStageColsD + cq * 32;
                const ulonglong2* sc = reinterpret_cast<const ulonglong2*>(smem + sm.s + bs * kStepBytesS) + cq * 16;
                uint64_t dd = 0ull;
                // two chunks of 16 columns: a round trip to tensor memory costs several hundred cycles
                // whatever its size, so few, large loads (as large as the registers allow)
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    uint32_t v0[16], v1[16];
                    if (c * 16 < ncols) {
                        tmem_ld16(t0 + c * 16, v0);
                        tmem_ld16(t0 + kTileTok + c * 16, v1);
                        tmem_ld_wait();
                    }
                    if (c == last_chunk) {
                        // all of this thread's sums are in registers: the tensor-memory stage goes back
                        // before the arithmetic on the last chunk; the stages limit the MMAs in flight
                        tc_fence_before_sync();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(bars + kBarDFree + ds);
                        d_ready = mbar_try_wait(bars + kBarDFull + (g + 1) % kStagesD, ((g + 1) / kStagesD) & 1u);
                    }
                    if (c == 0) {
                        if (!a_ready) a_ready = wait_full(kBarAFull + as, g / kStagesA);
                        if (!b_ready) b_ready = wait_full(kBarBFull + bs, g / kStagesB);
                        const float d = reinterpret_cast<const float*>(smem + sm.sw)[as * kTileRows + row];
                        dd = pack2(d, d);
                    }
                    if (c * 16 < ncols) {
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const ulonglong2 a = sc[c * 8 + i];   // {a0 of the two tokens}, {a1 of the two tokens}
                            const uint64_t s0 = pack2(__uint_as_float(v0[2 * i]), __uint_as_float(v0[2 * i + 1]));
                            const uint64_t s1 = pack2(__uint_as_float(v1[2 * i]), __uint_as_float(v1[2 * i + 1]));
                            // packed multiply by the row scale, then *scalar* adds: a packed add (or a
                            // packed t * 1 + acc) would be contracted with the multiply into one rounding
                            float u0, u1;
                            unpack2(mul2(dd, fma2(a.y, s1, mul2(a.x, s0))), u0, u1);
                            acc[c * 16 + 2 * i] = __fadd_rn(acc[c * 16 + 2 * i], u0);
                            acc[c * 16 + 2 * i + 1] = __fadd_rn(acc[c * 16 + 2 * i + 1], u1);
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(bars + kBarAFree + as);
                }
            }
            // ---- tile done: acc[i] holds this row's sum for token 32 cq + i
            if (GATE_UP) {
                // rows m < 8 of a group are gate rows, m >= 8 the up rows of the same ff rows: a
                // warp's 32 rows are 16 (gate, up) pairs, 128 contiguous bytes per token
                const int m = row & 15, ffrow = rb * 64 + (row >> 4) * 8 + (m & 7);
                float* dst = reinterpret_cast<float*>(p.hf) + size_t(ffrow) * 2 + (m >> 3);
#pragma unroll
                for (int i = 0; i < 32; ++i)
                    if (i < ncols) dst[size_t(p0 + 32 * cq + i) * p.ff * 2] = acc[i];
            } else {
                const int orow = rb * kTileRows + row;
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    if (2 * i < ncols) {
                        const float v0 = acc[2 * i], v1 = acc[2 * i + 1];
                        const int pos = p0 + 32 * cq + 2 * i;
                        const int sl0 = p.pslot[pos], sl1 = p.pslot[pos + 1];
                        if (p.y_bf16) {
                            __nv_bfloat16* yb = reinterpret_cast<__nv_bfloat16*>(p.yd);
                            if (sl0 >= 0) yb[size_t(sl0) * p.n + orow] = __float2bfloat16_rn(v0);
                            if (sl1 >= 0) yb[size_t(sl1) * p.n + orow] = __float2bfloat16_rn(v1);
                        } else {
                            if (sl0 >= 0) p.yd[size_t(sl0) * p.n + orow] = v0;
                            if (sl1 >= 0) p.yd[size_t(sl1) * p.n + orow] = v1;
                        }
                    }
                }
            }
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (*abort) {
        // A wait ran out: bulk copies and MMAs may still be in flight. Give them time to land
        // before tensor memory and the block's shared memory are released.
        const uint64_t t0 = global_ns();
        while (global_ns() - t0 < 2000000ull) {
        }
        __syncthreads();
    }
    if (warp == 1) tmem_free(tmem, 512);
    if (threadIdx.x == 0 && *abort) p.status[0] = kDevWaitTimeout;
}


int set_pf_attr() {
    static std::mutex mu;
    static bool done[64] = {};
    int dev = 0;
    FRX_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lk(mu);
    if (dev >= 0 && dev < 64 && done[dev]) return FRX_OK;
    FRX_CUDA(cudaFuncSetAttribute(k_pf_umma<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(pf_smem().total)));
    FRX_CUDA(cudaFuncSetAttribute(k_pf_umma<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(pf_smem().total)));
    if (dev >= 0 && dev < 64) done[dev] = true;
    return FRX_OK;
}

}  // namespace
}  // namespace frx

using namespace frx;

// The tensor-memory form pays per 128-row x 64-weight step whatever the number of tokens in the tile,
// so it is taken only when experts get many tokens on average.
constexpr int kUmmaMinTokensPerExpert = 256;

extern "C" {

// the streaming form lives in frx_decode.cu
size_t frx_moe_prefill_stream_workspace_bytes(int T, int K, int n, int ff, int E);
int frx_moe_prefill_stream_ex(const void* experts, size_t stride, int E, int n, int ff, const float* x, const int32_t* ids, int T, int K,
                              void* yd, void* ws, size_t ws_bytes, frx_stream_t stream, int block64, int yd_bf16);
int frx_moe_prefill_stream_q8_ep(const void* experts_local, size_t stride, int E_local, const int32_t* e_map, int E_all, int n, int ff,
                                 const int8_t* xq, const float* xd, const int32_t* ids, int T, int K, float* yd, void* ws, size_t ws_bytes,
                                 frx_stream_t stream);

size_t frx_moe_prefill_umma_workspace_bytes(int T, int K, int n, int ff, int E) {
    if (T < 1 || K < 1 || n < kUnitK || ff < kUnitK || E < 1) return 0;
    return pfu_layout(T, K, n, ff, E).total;
}

int frx_moe_prefill_umma(const void* experts, size_t stride, int E, int n, int ff, const float* x, const int32_t* ids, int T, int K,
                         float* yd, void* ws, size_t ws_bytes, frx_stream_t stream) {
    return frx_moe_prefill_umma_ex(experts, stride, E, n, ff, x, ids, T, K, yd, ws, ws_bytes, stream, 0, 0);
}

static int prefill_umma_impl(const void* experts, size_t stride, int E, const int32_t* e_map, int E_all, int n, int ff, const float* x,
                             const int8_t* xq_in, const float* xd_in, const int32_t* ids, int T, int K, void* yd, void* ws, size_t ws_bytes,
                             frx_stream_t stream, int block64, int yd_bf16) {
    if (!experts || !ids || !yd || !ws) return fail(FRX_ERR_ARG, "frx_moe_prefill: null pointer");
    if (n < kUnitK || ff < kUnitK || n % kUnitK || ff % kUnitK || n > 8192 || ff > 8192)
        return fail(FRX_ERR_SHAPE, "frx_moe_prefill: n %d and ff %d must be multiples of %d, at most 8192", n, ff, kUnitK);
    if (K < 1 || K > 32 || T < 0 || E < 1 || E > 4096 || E_all < E || E_all > 4096 || size_t(T) * K > (size_t(1) << 28))
        return fail(FRX_ERR_SHAPE, "frx_moe_prefill: unsupported T %d, K %d, E %d", T, K, E);
    if ((uintptr_t(experts) | stride) % 16 || uintptr_t(ws) % kAlign)
        return fail(FRX_ERR_ARG, "frx_moe_prefill: experts and stride must be 16-byte aligned, ws 256-byte aligned");
    if (stride < frx_q2_expert_bytes(n, ff)) return fail(FRX_ERR_ARG, "frx_moe_prefill: stride %zu < blob %zu", stride, frx_q2_expert_bytes(n, ff));
    if (T == 0) return FRX_OK;
    const PfuLayout L = pfu_layout(T, K, n, ff, E);
    if (ws_bytes < L.total) return fail(FRX_ERR_WORKSPACE, "frx_moe_prefill: workspace %zu < %zu", ws_bytes, L.total);
    if (int rc = set_pf_attr()) return rc;
    auto* base = static_cast<uint8_t*>(ws);
    int* status = reinterpret_cast<int*>(base + L.status);
    int* chunk_cnt = reinterpret_cast<int*>(base + L.chunk_cnt);
    int* bounds = reinterpret_cast<int*>(base + L.bounds);
    int* item_off = reinterpret_cast<int*>(base + L.item_off);
    int32_t* perm = reinterpret_cast<int32_t*>(base + L.perm);
    int* pb = reinterpret_cast<int*>(base + L.pb);
    int* tbo = reinterpret_cast<int*>(base + L.tbo);
    int* meta = reinterpret_cast<int*>(base + L.meta);
    int* tb_e = reinterpret_cast<int*>(base + L.tb_e);
    int* tb_p0 = reinterpret_cast<int*>(base + L.tb_p0);
    int* tb_n = reinterpret_cast<int*>(base + L.tb_n);
    int32_t* pslot = reinterpret_cast<int32_t*>(base + L.pslot);
    const int8_t* xq = xq_in ? xq_in : reinterpret_cast<const int8_t*>(base + L.xq);
    const float* xd = xd_in ? xd_in : reinterpret_cast<const float*>(base + L.xd);
    const int S = T * K;
    const size_t nblk = size_t(T) * (n / kQ8);
    if (!xq_in)   // else the activations arrived already quantized
        FRX_LAUNCH(kKQuant, stream, k_pfu_quant_x<<<unsigned((nblk + 7) / 8), 256, 0, stream>>>(x, nblk, reinterpret_cast<int8_t*>(base + L.xq),
                                                                                   reinterpret_cast<float*>(base + L.xd), block64));
    FRX_LAUNCH(kKGroup, stream, k_pf_hist<<<L.n_chunks, 256, size_t(E) * 4, stream>>>(ids, S, E, chunk_cnt, status, e_map, E_all));
    FRX_LAUNCH(kKGroup, stream, k_pf_scan<<<1, 1024, 0, stream>>>(chunk_cnt, L.n_chunks, E, bounds, item_off, status, 1 << 30));
    FRX_LAUNCH(kKGroup, stream, k_pf_place<<<L.n_chunks, 32, size_t(E) * 4, stream>>>(ids, S, E, chunk_cnt, bounds, perm, e_map, E_all));
    FRX_LAUNCH(kKGroup, stream, k_pfu_plan<<<1, 1024, 0, stream>>>(bounds, E, pb, tbo, meta, tb_e, tb_p0, tb_n, L.max_tb, status));
    FRX_LAUNCH(kKGroup, stream, k_pfu_gather<<<unsigned(L.pmax / 8), 256, 0, stream>>>(bounds, pb, E, perm, meta, K, n, L.pmax, xq, xd, base + L.xg,
                                                                                   reinterpret_cast<float*>(base + L.xa), pslot));
    UmmaParams p{};
    p.experts = static_cast<const uint8_t*>(experts);
    p.stride = stride;
    p.meta = meta;
    p.tb_e = tb_e;
    p.tb_p0 = tb_p0;
    p.tb_n = tb_n;
    p.pslot = pslot;
    p.hf = reinterpret_cast<float2*>(base + L.hf);
    p.yd = static_cast<float*>(yd);
    p.y_bf16 = yd_bf16 ? 1 : 0;
    p.status = status;
    p.pmax = L.pmax;
    p.wait_ns = wait_limit_ns();
    p.n = n;
    p.ff = ff;
    const int sms = sm_count();
    p.act = base + L.xg;
    p.act_scale = reinterpret_cast<const float*>(base + L.xa);
    FRX_LAUNCH(kKGateUp, stream, k_pf_umma<true><<<sms, kThreads, pf_smem().total, stream>>>(p));
    const size_t hchunks = L.pmax * size_t(ff / 8);
    FRX_LAUNCH(kKQuant, stream, k_pfu_quant_h<<<unsigned((hchunks + 255) / 256), 256, 0, stream>>>((const float2*)p.hf, ff, L.pmax, meta, pslot, base + L.hg,
                                                                                    reinterpret_cast<float*>(base + L.ha), block64));
    p.act = base + L.hg;
    p.act_scale = reinterpret_cast<const float*>(base + L.ha);
    FRX_LAUNCH(kKDown, stream, k_pf_umma<false><<<sms, kThreads, pf_smem().total, stream>>>(p));
    FRX_CUDA(cudaGetLastError());
    return FRX_OK;
}

int frx_moe_prefill_umma_ex(const void* experts, size_t stride, int E, int n, int ff, const float* x, const int32_t* ids, int T, int K,
                            void* yd, void* ws, size_t ws_bytes, frx_stream_t stream, int block64, int yd_bf16) {
    if (!x) return fail(FRX_ERR_ARG, "frx_moe_prefill: null pointer");
    return prefill_umma_impl(experts, stride, E, nullptr, E, n, ff, x, nullptr, nullptr, ids, T, K, yd, ws, ws_bytes, stream, block64, yd_bf16);
}

// ---- expert-parallel prefill on activations that arrive quantized: this rank holds E_local
// experts (e_map[id] = index here, or -1), the T tokens are all the tokens whose slots may land here
int frx_moe_prefill_q8_ep(const void* experts_local, size_t stride, int E_local, const int32_t* e_map, int E_all, int n, int ff,
                          const int8_t* xq, const float* xd, const int32_t* ids, int T, int K, float* yd, void* ws, size_t ws_bytes,
                          frx_stream_t stream, int form) {
    if (!xq || !xd || !e_map) return fail(FRX_ERR_ARG, "frx_moe_prefill_q8_ep: null pointer");
    if (form < 0 || form > 2) return fail(FRX_ERR_ARG, "frx_moe_prefill_q8_ep: form %d", form);
    // the expected number of slots per local expert is T * K / E_all (the counts stay on the device)
    const bool umma = form == 2 || (form == 0 && T > 0 && size_t(T) * K >= size_t(kUmmaMinTokensPerExpert) * size_t(E_all));
    if (umma) return prefill_umma_impl(experts_local, stride, E_local, e_map, E_all, n, ff, nullptr, xq, xd, ids, T, K, yd, ws, ws_bytes, stream, 0, 0);
    return frx_moe_prefill_stream_q8_ep(experts_local, stride, E_local, e_map, E_all, n, ff, xq, xd, ids, T, K, yd, ws, ws_bytes, stream);
}

// ---- the public entry. Both forms compute the same bits; the choice is by measured speed: the
// tensor-memory form pays per 128-row x 64-weight step whatever the number of tokens in the tile,
// so it is taken only when experts get many tokens on average (256 or more, where it is on a par
// with or ahead of the streaming form on B200), and the streaming form otherwise.

size_t frx_moe_prefill_workspace_bytes(int T, int K, int n, int ff, int E) {
    const size_t a = frx_moe_prefill_stream_workspace_bytes(T, K, n, ff, E), b = frx_moe_prefill_umma_workspace_bytes(T, K, n, ff, E);
    if (!a || !b) return 0;
    return a > b ? a : b;
}

int frx_moe_prefill(const void* experts, size_t stride, int E, int n, int ff, const float* x, const int32_t* ids, int T, int K,
                    float* yd, void* ws, size_t ws_bytes, frx_stream_t stream) {
    return frx_moe_prefill_ex(experts, stride, E, n, ff, x, ids, T, K, yd, ws, ws_bytes, stream, 0, 0);
}

int frx_moe_prefill_ex(const void* experts, size_t stride, int E, int n, int ff, const float* x, const int32_t* ids, int T, int K,
                       void* yd, void* ws, size_t ws_bytes, frx_stream_t stream, int block64, int yd_bf16) {
    if (T > 0 && K > 0 && E > 0 && size_t(T) * K >= size_t(kUmmaMinTokensPerExpert) * E)
        return frx_moe_prefill_umma_ex(experts, stride, E, n, ff, x, ids, T, K, yd, ws, ws_bytes, stream, block64, yd_bf16);
    return frx_moe_prefill_stream_ex(experts, stride, E, n, ff, x, ids, T, K, yd, ws, ws_bytes, stream, block64, yd_bf16);
}

}  // extern "C"
