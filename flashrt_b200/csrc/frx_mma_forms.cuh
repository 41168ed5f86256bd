// The inner products of the streaming expert kernels on the int8 tensor cores: one form for items
// of up to eight tokens and three for items of at most four, all with the same products, scaling
// and order of additions; and the build of a down item buffer from (gate x, up x) pairs. Include
// inside namespace frx { namespace { ... } } after the definition of Item.
#pragma once

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
