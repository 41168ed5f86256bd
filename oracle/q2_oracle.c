/*
 * CPU oracle for the Q2_0 MoE expert path: a scalar restatement of the reference's arithmetic.
 * TEST INFRASTRUCTURE ONLY (see q2_oracle.h). Build with -ffp-contract=off and without
 * -march=native: the reference's scalar float code is not contracted to FMA
 * (reference CMakeLists.txt:12-16), and bit-for-bit agreement depends on that.
 */
#include "q2_oracle.h"

#include <math.h>
#include <pthread.h>
#include <stdlib.h>
#include <string.h>

#define QK 64  /* weights per Q2_0 block      (quant/q2_0/q2_0.hpp:23) */
#define QB 18  /* bytes per block             (quant/q2_0/q2_0.hpp:24) */
#define Q8K 32 /* values per activation block (quant/q2_0/q2_0.hpp:25) */

/* ---- core/fp16.hpp:11-31: exact half -> float, subnormals normalised */
float orc_fp16_to_fp32(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu, man = h & 0x3ffu, bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {
            exp = 113;
            while (!(man & 0x400u)) {
                man <<= 1;
                --exp;
            }
            bits = sign | (exp << 23) | ((man & 0x3ffu) << 13);
        }
    } else if (exp == 0x1f) {
        bits = sign | 0x7f800000u | (man << 13);
    } else {
        bits = sign | ((exp + 112) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* ---- core/fp16.hpp:33-52: float -> half, round to nearest even */
uint16_t orc_fp32_to_fp16(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    const uint32_t sign = (x >> 16) & 0x8000u;
    const uint32_t a = x & 0x7fffffffu;
    if (a >= 0x7f800000u) return (uint16_t)(sign | 0x7c00u | (a > 0x7f800000u ? 0x200u : 0u));
    if (a >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u);
    if (a < 0x38800000u) {
        if (a < 0x33000000u) return (uint16_t)sign;
        const uint32_t e = a >> 23, m = (a & 0x7fffffu) | 0x800000u;
        const uint32_t shift = 126 - e;
        uint32_t h = m >> shift;
        const uint32_t rem = m & ((1u << shift) - 1), half = 1u << (shift - 1);
        if (rem > half || (rem == half && (h & 1u))) ++h;
        return (uint16_t)(sign | h);
    }
    uint32_t h = (a >> 13) - (112u << 10);
    const uint32_t rem = a & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (h & 1u))) ++h;
    return (uint16_t)(sign | h);
}

size_t orc_mat_bytes(int rows, int cols) { return (size_t)rows * (size_t)(cols / QK) * QB; }
size_t orc_expert_bytes(int n, int ff) { return 2 * orc_mat_bytes(ff, n) + orc_mat_bytes(n, ff); }

/* ---- quant/q2_0/q2_0.hpp:5-15: ggml element j of a block is in byte j/4 at bit 2*(j%4); the
 * planar block keeps it in byte j%16 at bit 2*(j/16). Codes first, then all fp16 scales. The
 * reference builds the same bytes through a 256-entry table (q2_0.cpp:25-39); tests pin both to
 * this element-wise placement (tests/test_q2_0.cpp:74-86). */
void orc_repack(const void* ggml_rows, int rows, int cols, void* dst) {
    const uint8_t* in = (const uint8_t*)ggml_rows;
    uint8_t* codes = (uint8_t*)dst;
    const size_t nblk = (size_t)rows * (size_t)(cols / QK);
    uint8_t* scales = codes + nblk * 16;
    for (size_t i = 0; i < nblk; ++i) {
        const uint8_t* b = in + i * QB; /* {uint16 d; uint8 qs[16]} */
        uint8_t o[16] = {0};
        for (int j = 0; j < QK; ++j) o[j % 16] |= (uint8_t)(((b[2 + j / 4] >> (2 * (j % 4))) & 3) << (2 * (j / 16)));
        memcpy(codes + i * 16, o, 16);
        memcpy(scales + i * 2, b, 2);
    }
}

void orc_repack_expert(const void* gate, const void* up, const void* down, int n, int ff, void* blob) {
    uint8_t* p = (uint8_t*)blob;
    const size_t gu = orc_mat_bytes(ff, n);
    orc_repack(gate, ff, n, p);
    orc_repack(up, ff, n, p + gu);
    orc_repack(down, n, ff, p + 2 * gu);
}

static inline int planar_code(const uint8_t* blk16, int j) { return (blk16[j % 16] >> (2 * (j / 16))) & 3; }

static inline uint16_t rd16(const uint8_t* p) {
    uint16_t v;
    memcpy(&v, p, 2);
    return v;
}

void orc_dequant_planar(const void* mat, int rows, int cols, float* out) {
    const uint8_t* codes = (const uint8_t*)mat;
    const int nb = cols / QK;
    const uint8_t* scales = codes + (size_t)rows * nb * 16;
    for (int r = 0; r < rows; ++r)
        for (int b = 0; b < nb; ++b) {
            const size_t k = (size_t)r * nb + b;
            const float d = orc_fp16_to_fp32(rd16(scales + 2 * k));
            for (int j = 0; j < QK; ++j) out[(size_t)r * cols + b * QK + j] = (float)(planar_code(codes + k * 16, j) - 1) * d;
        }
}

void orc_dequant_ggml(const void* ggml_rows, int rows, int cols, float* out) {
    const uint8_t* in = (const uint8_t*)ggml_rows;
    const int nb = cols / QK;
    for (int r = 0; r < rows; ++r)
        for (int b = 0; b < nb; ++b) {
            const uint8_t* blk = in + ((size_t)r * nb + b) * QB;
            const float d = orc_fp16_to_fp32(rd16(blk));
            for (int j = 0; j < QK; ++j)
                out[(size_t)r * cols + b * QK + j] = (float)(((blk[2 + j / 4] >> (2 * (j % 4))) & 3) - 1) * d;
        }
}

/* ---- quant/q2_0/q2_0.cpp:101-117 */
void orc_quantize_q8(const float* x, int n, int8_t* q, float* d) {
    for (int i = 0; i < n / Q8K; ++i) {
        const float* x32 = x + i * Q8K;
        float amax = 0.0f;
        for (int j = 0; j < Q8K; ++j) {
            const float a = fabsf(x32[j]);
            amax = amax < a ? a : amax; /* std::max(amax, |x|) */
        }
        const float dd = amax / 127.0f;
        const float id = dd != 0.0f ? 1.0f / dd : 0.0f;
        d[i] = orc_fp16_to_fp32(orc_fp32_to_fp16(dd));
        for (int j = 0; j < Q8K; ++j) q[i * Q8K + j] = (int8_t)roundf(x32[j] * id);
    }
}

/* ---- quant/q2_0/q2_0.cpp:119-140 */
void orc_matvec(const void* mat, int rows, int cols, const int8_t* q, const float* d, int r0, int r1, float* y) {
    const uint8_t* codes = (const uint8_t*)mat;
    const int nb = cols / QK;
    const uint8_t* scales = codes + (size_t)rows * nb * 16;
    for (int r = r0; r < r1; ++r) {
        float sumf = 0.0f;
        for (int b = 0; b < nb; ++b) {
            const uint8_t* blk = codes + ((size_t)r * nb + b) * 16;
            const float d0 = orc_fp16_to_fp32(rd16(scales + 2 * ((size_t)r * nb + b)));
            float sumi = 0.0f;
            for (int k = 0; k < 2; ++k) {
                int s = 0;
                for (int j = 0; j < Q8K; ++j) s += (planar_code(blk, k * Q8K + j) - 1) * q[b * QK + k * Q8K + j];
                sumi += d[2 * b + k] * (float)s;
            }
            sumf += d0 * sumi;
        }
        y[r] = sumf;
    }
}

/* ---- quant/q2_0/q2_0.cpp:142-158 */
float orc_dot_ggml(const void* ggml_row, int cols, const int8_t* q, const float* d) {
    const uint8_t* w = (const uint8_t*)ggml_row;
    float sumf = 0.0f;
    for (int b = 0; b < cols / QK; ++b) {
        const uint8_t* blk = w + (size_t)b * QB;
        const float d0 = orc_fp16_to_fp32(rd16(blk));
        float sumi = 0.0f;
        for (int k = 0; k < 2; ++k) {
            int s = 0;
            for (int i = 0; i < 8; ++i) {
                const uint8_t byte = blk[2 + k * 8 + i];
                for (int e = 0; e < 4; ++e) s += (((byte >> (2 * e)) & 3) - 1) * q[b * QK + k * Q8K + 4 * i + e];
            }
            sumi += d[2 * b + k] * (float)s;
        }
        sumf += d0 * sumi;
    }
    return sumf;
}

/* ---- quant/q2_0/q2_0.cpp:160-185, one token, scalar matvec */
void orc_expert_ffn(const void* blob, int n, int ff, const int8_t* xq, const float* xd, float* out, float* h, int8_t* hq,
                    float* hd) {
    const uint8_t* p = (const uint8_t*)blob;
    const size_t gu = orc_mat_bytes(ff, n);
    float* g = (float*)malloc(sizeof(float) * (size_t)ff * 2);
    float* u = g + ff;
    int8_t* q = hq ? hq : (int8_t*)malloc((size_t)ff);
    float* d = hd ? hd : (float*)malloc(sizeof(float) * (size_t)(ff / Q8K));
    orc_matvec(p, ff, n, xq, xd, 0, ff, g);
    orc_matvec(p + gu, ff, n, xq, xd, 0, ff, u);
    for (int i = 0; i < ff; ++i) g[i] = g[i] / (1.0f + expf(-g[i])) * u[i];
    if (h) memcpy(h, g, sizeof(float) * (size_t)ff);
    orc_quantize_q8(g, ff, q, d);
    orc_matvec(p + 2 * gu, n, ff, q, d, 0, n, out);
    free(g);
    if (!hq) free(q);
    if (!hd) free(d);
}

/* ---- arch/qwen4exp/moe_ref.cu:150-170. std::partial_sort leaves the order of equal
 * probabilities unspecified; the reference's GPU router and its test fix it as "ties to the lower
 * index" (moe_ref.cu:51-61, tests/test_route_topk.cpp:52-55), which is what this does. */
void orc_route(const float* logits, int T, int E, int K, int32_t* ids, float* wts, float* probs) {
    float* p = (float*)malloc(sizeof(float) * (size_t)E);
    for (int t = 0; t < T; ++t) {
        const float* lg = logits + (size_t)t * E;
        float mx = lg[0];
        for (int e = 1; e < E; ++e) mx = mx < lg[e] ? lg[e] : mx;
        double sum = 0;
        for (int e = 0; e < E; ++e) sum += p[e] = expf(lg[e] - mx);
        for (int e = 0; e < E; ++e) p[e] = (float)(p[e] / sum);
        int32_t* id = ids + (size_t)t * K;
        for (int k = 0; k < K; ++k) {
            int best = -1;
            for (int e = 0; e < E; ++e) {
                int taken = 0;
                for (int j = 0; j < k; ++j) taken |= id[j] == e;
                if (!taken && (best < 0 || p[e] > p[best])) best = e;
            }
            id[k] = best;
        }
        float wsum = 0.0f;
        for (int k = 0; k < K; ++k) wsum += p[id[k]];
        wsum = wsum < 6.103515625e-5f ? 6.103515625e-5f : wsum;
        for (int k = 0; k < K; ++k) {
            wts[(size_t)t * K + k] = p[id[k]] / wsum;
            if (probs) probs[(size_t)t * K + k] = p[id[k]];
        }
    }
    free(p);
}

/* A small parallel-for over expert evaluations; results do not depend on the thread count. */
typedef struct {
    const uint8_t* experts;
    size_t stride;
    const uint8_t* shared;
    int n, ff, K, S;
    const int8_t* xq;
    const float* xd;
    const int32_t* ids;
    float* ys;
    int next;
    pthread_mutex_t mu;
} FfnJob;

static void* ffn_worker(void* arg) {
    FfnJob* j = (FfnJob*)arg;
    for (;;) {
        pthread_mutex_lock(&j->mu);
        const int s = j->next++;
        pthread_mutex_unlock(&j->mu);
        if (s >= j->S) return NULL;
        const int t = j->shared ? s : s / j->K;
        const uint8_t* blob = j->shared ? j->shared : j->experts + (size_t)j->ids[s] * j->stride;
        orc_expert_ffn(blob, j->n, j->ff, j->xq + (size_t)t * j->n, j->xd + (size_t)t * (j->n / Q8K), j->ys + (size_t)s * j->n,
                       NULL, NULL, NULL);
    }
}

static void run_ffn_job(FfnJob* j, int n_threads) {
    pthread_t th[64];
    if (n_threads > 64) n_threads = 64;
    j->next = 0;
    pthread_mutex_init(&j->mu, NULL);
    for (int i = 1; i < n_threads; ++i) pthread_create(&th[i], NULL, ffn_worker, j);
    ffn_worker(j);
    for (int i = 1; i < n_threads; ++i) pthread_join(th[i], NULL);
    pthread_mutex_destroy(&j->mu);
}

/* ---- arch/qwen4exp/moe_ref.cu:138-188 with quant/q2_0/moe_cpu.cpp:36-81.
 * moe_cpu adds the experts' outputs into a zeroed row in entry order; entries are built in
 * ascending expert id, each holding the expert's tokens in token order (moe_ref.cu:171-183), so a
 * token's sum runs over its experts in ascending id: out = ((0 + w0*y0) + w1*y1) + ...
 * The shared expert follows k_add_gated (moe_ref.cu:91-97): out = moe + shexp * g,
 * g = 1 / (1 + exp(-gate)). */
void orc_moe_layer(const uint8_t* experts, size_t stride, const uint8_t* shared, int n, int ff, const float* x, int T,
                   const int32_t* ids, const float* wts, int K, const float* gate_logit, float* out, float* yslot,
                   float* ysh, int n_threads) {
    int8_t* xq = (int8_t*)malloc((size_t)T * n);
    float* xd = (float*)malloc(sizeof(float) * (size_t)T * (n / Q8K));
    for (int t = 0; t < T; ++t) orc_quantize_q8(x + (size_t)t * n, n, xq + (size_t)t * n, xd + (size_t)t * (n / Q8K));
    float* ys = yslot ? yslot : (float*)malloc(sizeof(float) * (size_t)T * K * n);
    FfnJob job = {experts, stride, NULL, n, ff, K, T * K, xq, xd, ids, ys, 0, PTHREAD_MUTEX_INITIALIZER};
    run_ffn_job(&job, n_threads);
    int* order = (int*)malloc(sizeof(int) * (size_t)K);
    for (int t = 0; t < T; ++t) {
        for (int k = 0; k < K; ++k) order[k] = k;
        for (int a = 1; a < K; ++a) /* ascending expert id */
            for (int b = a; b > 0 && ids[t * K + order[b - 1]] > ids[t * K + order[b]]; --b) {
                const int tmp = order[b];
                order[b] = order[b - 1];
                order[b - 1] = tmp;
            }
        float* o = out + (size_t)t * n;
        for (int r = 0; r < n; ++r) o[r] = 0.0f;
        for (int k = 0; k < K; ++k) {
            const float w = wts[t * K + order[k]];
            const float* y = ys + (size_t)(t * K + order[k]) * n;
            for (int r = 0; r < n; ++r) o[r] += w * y[r];
        }
    }
    free(order);
    if (shared) {
        float* sh = ysh ? ysh : (float*)malloc(sizeof(float) * (size_t)T * n);
        FfnJob sjob = {NULL, 0, shared, n, ff, 1, T, xq, xd, NULL, sh, 0, PTHREAD_MUTEX_INITIALIZER};
        run_ffn_job(&sjob, n_threads);
        for (int t = 0; t < T; ++t) {
            const float g = gate_logit ? 1.0f / (1.0f + expf(-gate_logit[t])) : 1.0f;
            for (int r = 0; r < n; ++r) out[(size_t)t * n + r] = out[(size_t)t * n + r] + sh[(size_t)t * n + r] * g;
        }
        if (!ysh) free(sh);
    }
    if (!yslot) free(ys);
    free(xq);
    free(xd);
}

/* The layer join of the chained expert-stack benchmark (no reference counterpart: the benchmark
 * definition itself): out = r / sqrt(mean(r^2) + 1e-6), r = x + y, with the operation order of the
 * GPU kernel: 32 partial sums of squares in double, partial l over elements l, l + 32, ... in
 * that order, combined by a butterfly (offsets 16, 8, 4, 2, 1), then one double division and
 * square root, the factor rounded to float. */
void orc_chain_rmsnorm_unit(const float* x, const float* y, float* out, int T, int n) {
    for (int t = 0; t < T; ++t) {
        const float* xr = x + (size_t)t * n;
        const float* yr = y + (size_t)t * n;
        double part[32];
        for (int l = 0; l < 32; ++l) {
            double ss = 0.0;
            for (int i = l; i < n; i += 32) {
                const float r = xr[i] + yr[i];
                ss += (double)r * (double)r;
            }
            part[l] = ss;
        }
        for (int o = 16; o > 0; o >>= 1) {
            double nxt[32];
            for (int l = 0; l < 32; ++l) nxt[l] = part[l] + part[l ^ o];
            memcpy(part, nxt, sizeof part);
        }
        const float inv = (float)(1.0 / sqrt(part[0] / (double)n + 1e-6));
        for (int i = 0; i < n; ++i) out[(size_t)t * n + i] = (xr[i] + yr[i]) * inv;
    }
}
