/*
 * CPU oracle for the ggml-layout entry points of the Q2_0 expert path (the reference's
 * kernels/cuda/ggml_gemv.h and ggml_gemm.h, which run llama.cpp's kernels vendored under
 * third_party/ggml) and for the Q8_0 -> Q2_0 requantizer of its draft head.
 * TEST INFRASTRUCTURE ONLY (see q2_oracle.h): nothing in the product links or calls this file.
 *
 * What is pinned and what is not. The activation quantizer (Q8_1) and the requantizer are
 * restated operation for operation and are compared bit for bit. The dot product follows
 * vec_dot_q2_0_q8_1 per 32-value chunk exactly (integer sum, then d2 * d8 * sumi in float); the
 * order in which ggml adds the chunks of a row depends on its launch shape (threads stride over
 * blocks, then a shuffle tree), so the chunk values are added here in double and results are
 * compared within the tolerance the reference's own test uses for this path
 * (tests/test_moe_q.cpp:7-9: 1e-4 relative).
 */
#include "q2_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

#define QK 64
#define QB 18
#define Q81 36 /* block_q8_1: half d, half s, 32 int8 (third_party/ggml/src/ggml-common.h:256-268) */

/* third_party/ggml/src/ggml-cuda/quantize.cu:54-101 (quantize_q8_1) as called by gemv::quantize_q8_1
 * (kernels/cuda/ggml_gemv.cu:82-87): rows padded with zeros to a multiple of 512 values; per 32
 * values d = amax / 127, q = amax == 0 ? 0 : roundf(x / d); the block keeps half(d) and
 * half(sum of the 32 inputs). The sum is added here in index order; the GPU adds it by a
 * shuffle tree, so `s` may differ in its last fp16 bit (the Q2_0 dot does not read it). */
void orc_quantize_q8_1(const float* x, int ncols, int n_tok, uint8_t* out) {
    const int padded = (ncols + 511) / 512 * 512;
    for (int t = 0; t < n_tok; ++t)
        for (int b = 0; b < padded / 32; ++b) {
            float v[32], amax = 0.0f, sum = 0.0f;
            for (int i = 0; i < 32; ++i) {
                const int c = b * 32 + i;
                v[i] = c < ncols ? x[(size_t)t * ncols + c] : 0.0f;
                amax = fmaxf(amax, fabsf(v[i]));
                sum += v[i];
            }
            const float d = amax / 127.0f;
            uint8_t* blk = out + ((size_t)t * (padded / 32) + b) * Q81;
            const uint16_t dh = orc_fp32_to_fp16(d), sh = orc_fp32_to_fp16(sum);
            memcpy(blk, &dh, 2);
            memcpy(blk + 2, &sh, 2);
            for (int i = 0; i < 32; ++i) blk[4 + i] = (uint8_t)(int8_t)(amax == 0.0f ? 0 : (int)roundf(v[i] / d));
        }
}

/* third_party/ggml/src/ggml-cuda/vecdotq.cuh:728-771 (vec_dot_q2_0_q8_1): one 32-value chunk of a
 * Q2_0 block against one Q8_1 block: sumi = sum (q - 1) * a, value = d2 * d8 * sumi (float).
 * Element j of the block is in byte j / 4 at bit 2 * (j % 4). */
static float chunk_q2_0_q8_1(const uint8_t* wblk, int chunk, const uint8_t* ablk) {
    uint16_t dh, ah;
    memcpy(&dh, wblk, 2);
    memcpy(&ah, ablk, 2);
    const float d2 = orc_fp16_to_fp32(dh), d8 = orc_fp16_to_fp32(ah);
    const int8_t* a = (const int8_t*)(ablk + 4);
    int sumi = 0;
    for (int i = 0; i < 32; ++i) {
        const int j = chunk * 32 + i;
        const int q = (wblk[2 + j / 4] >> (2 * (j % 4))) & 3;
        sumi += (q - 1) * a[i];
    }
    return d2 * d8 * (float)sumi;
}

/* One row of ggml Q2_0 blocks against one row of Q8_1 blocks; chunk values added in double. */
double orc_dot_q2_0_q8_1(const uint8_t* wrow, int ncols, const uint8_t* xq_row) {
    double acc = 0.0;
    for (int b = 0; b < ncols / QK; ++b)
        for (int c = 0; c < 2; ++c) acc += (double)chunk_q2_0_q8_1(wrow + (size_t)b * QB, c, xq_row + (size_t)(2 * b + c) * Q81);
    return acc;
}

/* gemv::moe_q for Q2_0 (kernels/cuda/ggml_gemv.h:56-65): dst[t][j][r] = W_e row r . x, e = ids[t][j],
 * W_e at w + e * expert_stride; x = Q8_1 row t (or row t * k + j with act_per_expert); with gate,
 * silu(G_e row r . x) * (W_e row r . x), silu(g) = g / (1 + expf(-g)) (ggml unary.cuh:98-100). */
void orc_moe_q2_0(const uint8_t* w, const uint8_t* gate, const uint8_t* xq, const int32_t* ids, float* dst, int n_tok, int k, int ncols,
                  int nrows, size_t expert_stride, int act_per_expert) {
    const size_t act_row = (size_t)((ncols + 511) / 512 * 512 / 32) * Q81, wrow = (size_t)(ncols / QK) * QB;
    for (int t = 0; t < n_tok; ++t)
        for (int j = 0; j < k; ++j) {
            const int e = ids[t * k + j];
            const uint8_t* a = xq + (size_t)(act_per_expert ? t * k + j : t) * act_row;
            for (int r = 0; r < nrows; ++r) {
                float v = (float)orc_dot_q2_0_q8_1(w + (size_t)e * expert_stride + (size_t)r * wrow, ncols, a);
                if (gate) {
                    const float g = (float)orc_dot_q2_0_q8_1(gate + (size_t)e * expert_stride + (size_t)r * wrow, ncols, a);
                    v = g / (1.0f + expf(-g)) * v;
                }
                dst[((size_t)t * k + j) * nrows + r] = v;
            }
        }
}

/* The Q8_0 -> Q2_0 conversion of the draft head as first written, which the reference's test keeps
 * as its golden form (tests/test_mtp_convert.cu:34-62; the shipped form, arch/qwen4exp/mtp.cu:129-201,
 * must equal it bit for bit): 64 values from two Q8_0 blocks {fp16 d; 32 int8}, 24 candidate
 * scales from amax / 2.5 up to amax (through fp16), codes clamp(lround(x / d), -1, 2), the
 * candidate with the smallest squared error (added in index order, first minimum wins).
 * lround of a non-finite value is taken as 0, which is what the reference's build does on x86-64
 * (the conversion returns the "indefinite" integer, whose low 32 bits are zero). */
static int q2_round(float v) {
    if (!isfinite(v)) return 0;
    const long r = lroundf(v);
    return (int)(r < -1 ? -1 : r > 2 ? 2 : r);
}
void orc_convert_q8_0_to_q2_0(const uint8_t* src, uint8_t* dst, size_t nblocks64) {
    for (size_t b = 0; b < nblocks64; ++b, src += 68, dst += 18) {
        float x[64], amax = 0.0f;
        for (int h = 0; h < 2; ++h) {
            const uint8_t* s8 = src + 34 * h;
            uint16_t dh;
            memcpy(&dh, s8, 2);
            const float d8 = orc_fp16_to_fp32(dh);
            for (int j = 0; j < 32; ++j) {
                x[32 * h + j] = d8 * (float)(int8_t)s8[2 + j];
                amax = fmaxf(amax, fabsf(x[32 * h + j]));
            }
        }
        float best_d = 0.0f, best_e = INFINITY;
        for (int c = 0; c < 24 && amax > 0.0f; ++c) {
            const float d = amax / (2.5f - 1.5f * (float)c / 23.0f);
            const float dq = orc_fp16_to_fp32(orc_fp32_to_fp16(d));
            float e = 0.0f;
            for (int j = 0; j < 64; ++j) {
                const int q = q2_round(x[j] / dq);
                const float r = x[j] - (float)q * dq;
                e += r * r;
            }
            if (e < best_e) {
                best_e = e;
                best_d = dq;
            }
        }
        const uint16_t dh = orc_fp32_to_fp16(best_d);
        memcpy(dst, &dh, 2);
        memset(dst + 2, 0, 16);
        for (int j = 0; j < 64; ++j) {
            const int q = best_d > 0.0f ? q2_round(x[j] / best_d) : 0;
            dst[2 + j / 4] |= (uint8_t)((q + 1) << (2 * (j % 4)));
        }
    }
}
