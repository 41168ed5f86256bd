/*
 * CPU oracle for the Q2_0 MoE expert path. TEST INFRASTRUCTURE ONLY: nothing in the product
 * (the flashrt_b200 package or libfrx) may link, import or call this file. It is used by the
 * parity tests, the smoke check and the CPU-baseline leg of the benchmark.
 *
 * Each function restates, in plain scalar C, the arithmetic of one function of the reference
 * (flashrt), in the same order of floating-point operations, so results can be compared bit for
 * bit. The reference file:line each one follows is given beside it in q2_oracle.c.
 *
 * Parity is pinned: tests/test_oracle_pins.py checks these functions against the reference's own
 * known-answer values, and tests/test_oracle_vs_ref.py checks them against the reference sources
 * compiled unmodified (oracle/_ref) on seeded inputs.
 */
#ifndef Q2_ORACLE_H
#define Q2_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* core/fp16.hpp:11-52 */
float orc_fp16_to_fp32(uint16_t h);
uint16_t orc_fp32_to_fp16(float f);

/* quant/q2_0/q2_0.cpp:43,66 */
size_t orc_mat_bytes(int rows, int cols);
size_t orc_expert_bytes(int n, int ff);

/* quant/q2_0/q2_0.cpp:34-39,51-80: ggml blocks {fp16 d; 16 code bytes} -> planar matrix */
void orc_repack(const void* ggml_rows, int rows, int cols, void* dst);
void orc_repack_expert(const void* gate, const void* up, const void* down, int n, int ff, void* blob);

/* (q - 1) * fp16_to_fp32(d) for every weight of a planar / ggml matrix, row-major [rows][cols] */
void orc_dequant_planar(const void* mat, int rows, int cols, float* out);
void orc_dequant_ggml(const void* ggml_rows, int rows, int cols, float* out);

/* quant/q2_0/q2_0.cpp:101-117: per 32 values; q [n] int8, d [n/32] (fp16-rounded, as float) */
void orc_quantize_q8(const float* x, int n, int8_t* q, float* d);

/* quant/q2_0/q2_0.cpp:119-140 (matvec_ref): y[r] for r in [r0, r1) of one planar matrix */
void orc_matvec(const void* mat, int rows, int cols, const int8_t* q, const float* d, int r0, int r1, float* y);
/* quant/q2_0/q2_0.cpp:142-158 (dot_ggml) on ggml-order blocks of one row */
float orc_dot_ggml(const void* ggml_row, int cols, const int8_t* q, const float* d);

/* quant/q2_0/q2_0.cpp:160-185 (expert_ffn, scalar path) for one token.
 * Optional outputs (may be NULL): h [ff] fp32 hidden, hq [ff] / hd [ff/32] its Q8 form. */
void orc_expert_ffn(const void* blob, int n, int ff, const int8_t* xq, const float* xd, float* out, float* h, int8_t* hq,
                    float* hd);

/* arch/qwen4exp/moe_ref.cu:150-170: softmax (float exp, double sum), top-K by probability
 * (ties to the lower index), weights p / max(sum of selected, 6.103515625e-5).
 * ids, wts [T][K]; probs [T][K] optional. */
void orc_route(const float* logits, int T, int E, int K, int32_t* ids, float* wts, float* probs);

/* One MoE layer as moe_block + moe_cpu compute it (arch/qwen4exp/moe_ref.cu:138-188,
 * quant/q2_0/moe_cpu.cpp:36-81): per-token Q8 of x, experts visited in ascending id and token
 * order, out[t] = sum_e w * expert_e(x_t) accumulated in that order, then
 * out += shexp * sigmoid(gate) when a shared expert is given.
 *   experts: planar blobs at experts + e * stride; shared: one planar blob or NULL;
 *   x [T][n]; ids, wts [T][K]; gate_logit [T] or NULL (then the shared expert's weight is 1);
 *   out [T][n]; yslot [T*K][n] optional per-slot expert outputs (slot t*K+k);
 *   ysh [T][n] optional shared-expert outputs.
 * n_threads > 1 spreads the expert evaluations over POSIX threads; the result does not depend on it. */
void orc_moe_layer(const uint8_t* experts, size_t stride, const uint8_t* shared, int n, int ff, const float* x, int T,
                   const int32_t* ids, const float* wts, int K, const float* gate_logit, float* out, float* yslot,
                   float* ysh, int n_threads);

/* The layer join of the chained expert-stack benchmark: out[t] = r / sqrt(mean(r^2) + 1e-6), r = x[t] + y[t],
 * in the operation order of the GPU kernel (bit-identical). */
void orc_chain_rmsnorm_unit(const float* x, const float* y, float* out, int T, int n);

/* ---- ggml-layout pieces (ggml_oracle.c) ---- */

/* third_party/ggml/src/ggml-cuda/quantize.cu:54-101 as called by kernels/cuda/ggml_gemv.cu:82-87:
 * x [n_tok][ncols] -> Q8_1 rows of 36-byte blocks {fp16 d; fp16 sum; 32 int8}, rows padded with
 * zeros to a multiple of 512 values. */
void orc_quantize_q8_1(const float* x, int ncols, int n_tok, uint8_t* out);
/* third_party/ggml/src/ggml-cuda/vecdotq.cuh:728-771: one row of ggml Q2_0 blocks against one
 * Q8_1 row; the per-chunk values d2 * d8 * sumi (float) are added in double. */
double orc_dot_q2_0_q8_1(const uint8_t* wrow, int ncols, const uint8_t* xq_row);
/* kernels/cuda/ggml_gemv.h:56-65 (gemv::moe_q) for Q2_0 */
void orc_moe_q2_0(const uint8_t* w, const uint8_t* gate, const uint8_t* xq, const int32_t* ids, float* dst, int n_tok, int k, int ncols,
                  int nrows, size_t expert_stride, int act_per_expert);
/* tests/test_mtp_convert.cu:34-62, arch/qwen4exp/mtp.cu:129-201: Q8_0 block pairs -> ggml Q2_0 blocks */
void orc_convert_q8_0_to_q2_0(const uint8_t* src, uint8_t* dst, size_t nblocks64);

#ifdef __cplusplus
}
#endif
#endif
