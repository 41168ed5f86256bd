// Shared definitions for the libfrx kernels (sm_100a only).
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

#include "frx.h"

namespace frx {

// ---- Q2_0 format and the tiled layout (see frx_q2_tile_experts in frx.h)
constexpr int kQK = 64;           // weights per Q2_0 block
constexpr int kBlockBytes = 18;   // fp16 scale + 16 code bytes
constexpr int kQ8 = 32;           // values per int8 activation block
constexpr int kUnitRows = 16;     // M rows of one unit
constexpr int kUnitK = 128;       // weights of K in one unit (two blocks)
constexpr int kUnitCodeBytes = 512;
constexpr int kUnitBytes = 576;   // 16 rows x 2 blocks x 18 bytes
constexpr int kTokPerItem = 8;    // tokens of one work item: the N of mma.m16n8k32

// The float 1.5 * 2^23 and its bit pattern: an int32 accumulator started at kMagicBits + c,
// read as a float, is exactly kMagic + c for |c| < 2^22, so int -> float costs one subtraction.
constexpr float kMagic = 12582912.0f;
constexpr int kMagicBits = 0x4B400000;

constexpr size_t kAlign = 256;
__host__ __device__ inline size_t align_up(size_t x, size_t a = kAlign) { return (x + a - 1) / a * a; }

inline size_t gu_group_bytes(int n) { return size_t(n / kUnitK) * kUnitBytes; }      // 8 gate + 8 up rows
inline size_t down_group_bytes(int ff) { return size_t(ff / kUnitK) * kUnitBytes; }  // 16 down rows
inline size_t gu_section_bytes(int n, int ff) { return size_t(ff / 8) * gu_group_bytes(n); }

// ---- errors (host side)
int fail(int code, const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);
#define FRX_CUDA(expr)                                              \
    do {                                                            \
        cudaError_t e_ = (expr);                                    \
        if (e_ != cudaSuccess) return ::frx::cuda_fail(e_, #expr);  \
    } while (0)

int sm_count();
int max_smem_optin();

// Optional per-kernel timing (frx_profile_begin / frx_profile_end): when switched on, every
// launch made through FRX_LAUNCH is bracketed by two CUDA events on its own stream.
enum KernelClass : int { kKRoute = 0, kKQuant, kKGroup, kKGateUp, kKDown, kKCombine, kKLayout, kKPrologue, kKFfn, kNumKernelClasses };
extern bool g_profile_on;
void profile_mark(int cls, cudaStream_t stream, bool start);
#define FRX_LAUNCH(cls, stream, ...)                                   \
    do {                                                               \
        if (::frx::g_profile_on) ::frx::profile_mark(cls, stream, true);  \
        __VA_ARGS__;                                                   \
        if (::frx::g_profile_on) ::frx::profile_mark(cls, stream, false); \
    } while (0)

// Programmatic dependent launch: a kernel launched with launch_pdl may begin (be scheduled, run its
// prologue) while the kernel before it in the stream is still running; it must call pdl_wait()
// before it reads or writes anything the earlier kernels touch. pdl_wait() returns once those
// kernels have completed and their writes are visible; without the launch attribute it is a no-op.
// Every kernel of a chain calls it first thing, so completion is transitive along the chain.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <class... KArgs, class... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// The same with thread-block clusters of `cluster` blocks along x (grid.x a multiple of it).
template <class... KArgs, class... Args>
inline cudaError_t launch_pdl_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, unsigned cluster,
                                      Args... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2]{};
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = cluster;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t cluster_id_x() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%clusterid.x;" : "=r"(r));
    return r;
}
// Hardware barrier over all threads of the cluster; writes made before it (global memory
// included) are visible to the cluster's threads after it.
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Device-side error codes written to a workspace's status word.
enum : int {
    kDevOk = 0,
    kDevBadExpertId = 1,   // an id outside [0, E)
    kDevWaitTimeout = 2,   // a bounded wait on a shared-memory barrier ran out
    kDevTooManyItems = 3,
};

// ---- PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return uint32_t(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Non-blocking test of a barrier phase.
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ uint64_t global_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Waits for a barrier phase for at most limit_ns. Returns false when the wait ran out or
// `*abort` was already set; it then sets `*abort` so every later wait of the block returns at
// once, and the caller's block finishes its control flow without trusting the data.
// The limit is a launch parameter: wait_limit_ns() on the host, 2 s unless
// frx_debug_set_wait_limit_ns has changed it (tests shorten it to exercise the give-up paths).
constexpr uint64_t kWaitLimitNs = 2000000000ull;
uint64_t wait_limit_ns();
// SLEEP: back off with nanosleep after a few polls (right for waits on data from global memory,
// where a waiting warp should leave the issue slots to working warps); without it the wait only
// repeats try_wait, which itself suspends the thread for a short hardware-defined time (right for
// the short hand-offs of a warp-specialised pipeline, where a sleep that overshoots delays every step).
template <bool SLEEP = true>
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, volatile int* abort, uint64_t limit_ns) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*abort) return false;
    uint64_t t0 = 0;   // the clock is only read once the wait has lasted a while: reading it is slow
    for (uint32_t polls = 1;; ++polls) {
        if (mbar_try_wait(bar, parity)) return true;   // suspends the thread for a short, hardware-defined time when not complete
        if (SLEEP) {
            if (polls > 4) __nanosleep(polls > 64 ? 256 : 32);   // a long wait must not take issue slots from working warps
        } else if (polls > 65536) {
            __nanosleep(64);
        }
        if ((polls & 63u) == 0) {
            if (*abort) return false;
            const uint64_t now = global_ns();
            if (t0 == 0) {
                t0 = now;
            } else if (now - t0 > limit_ns) {
                *abort = 1;
                return false;
            }
        }
    }
}

// Touches the line at p without using it: the address translation (and the line in the L2) is there
// by the time a dependent access needs it. Used before griddepcontrol.wait, on buffers whose
// first access would otherwise pay a translation miss in the middle of a latency chain.
__device__ __forceinline__ void touch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }

// Counters in global memory that blocks of one grid raise and await.
__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void red_release_gpu_add(int* p, int v) {
    asm volatile("red.release.gpu.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// 1-D bulk copy global -> shared through the TMA unit, completion counted on an mbarrier.
// dst, src 16-byte aligned; bytes a multiple of 16.
// The same with an L2 eviction policy for the lines the copy brings in (see l2_policy_evict_first).
__device__ __forceinline__ void bulk_g2s_hint(void* dst, const void* src, uint32_t bytes, uint64_t* bar, uint64_t policy) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(
                     smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
                 : "memory");
}
// Policy for data that is read once (a decode step's expert weights: 326 MB per layer through a
// 126 MB L2): its lines are the first to go, so the stream does not push out what is read again
// (the next kernels' code, item lists, activations).
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
    return policy;
}
__device__ __forceinline__ uint64_t l2_policy_evict_normal() {   // the default behaviour, as a policy operand
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_normal.b64 %0, 1.0;" : "=l"(policy));
    return policy;
}
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// Non-blocking arrival at a hardware barrier that other threads bar.sync on.
__device__ __forceinline__ void named_bar_arrive(int id, int threads) {
    asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
__device__ __forceinline__ void named_bar_sync(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// D (16x8 s32) += A (16x32 u8, row) * B (32x8 s8, col)
__device__ __forceinline__ void mma_u8s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// D (16x8 s32) = A * B + C with every element of C equal to `c`; the results come back packed in
// pairs: lo = {D[g][2t], D[g][2t+1]}, hi = the same columns of row g + 8.
// The same with the accumulator input given as four registers (a quad loaded from shared memory).
__device__ __forceinline__ void mma_u8s8_c4(uint64_t& lo, uint64_t& hi, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                            uint32_t b1, const int4& c) {
    asm volatile(
        "{\n\t.reg .b32 d0, d1, d2, d3;\n\t"
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {d0,d1,d2,d3}, {%2,%3,%4,%5}, {%6,%7}, {%8,%9,%10,%11};\n\t"
        "mov.b64 %0, {d0,d1};\n\t"
        "mov.b64 %1, {d2,d3};\n\t}"
        : "=l"(lo), "=l"(hi)
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(c.x), "r"(c.y), "r"(c.z), "r"(c.w));
}

// Two MMAs chained into one accumulator: D = A0 * B0 + A1 * B1 + C with every element of C equal
// to `c`, results packed as above. Used with B operands that are zero in complementary token
// columns, so that the columns of D belong to different row groups.
__device__ __forceinline__ void mma_u8s8_chain2(uint64_t& lo, uint64_t& hi, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                uint32_t b0, uint32_t b1, uint32_t e0, uint32_t e1, uint32_t e2, uint32_t e3,
                                                uint32_t f0, uint32_t f1, int c) {
    asm volatile(
        "{\n\t.reg .b32 d0, d1, d2, d3;\n\t"
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {d0,d1,d2,d3}, {%2,%3,%4,%5}, {%6,%7}, {%14,%14,%14,%14};\n\t"
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {d0,d1,d2,d3}, {%8,%9,%10,%11}, {%12,%13}, {d0,d1,d2,d3};\n\t"
        "mov.b64 %0, {d0,d1};\n\t"
        "mov.b64 %1, {d2,d3};\n\t}"
        : "=l"(lo), "=l"(hi)
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(e0), "r"(e1), "r"(e2), "r"(e3), "r"(f0), "r"(f1), "r"(c));
}

// Four MMAs chained into one accumulator (see mma_u8s8_chain2): D = sum_j A_j * B_j + C.
__device__ __forceinline__ void mma_u8s8_chain4(uint64_t& lo, uint64_t& hi, const uint32_t (&a)[16], const uint32_t (&b)[8], int c) {
    asm volatile(
        "{\n\t.reg .b32 d0, d1, d2, d3;\n\t"
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {d0,d1,d2,d3}, {%2,%3,%4,%5}, {%18,%19}, {%26,%26,%26,%26};\n\t"
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {d0,d1,d2,d3}, {%6,%7,%8,%9}, {%20,%21}, {d0,d1,d2,d3};\n\t"
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {d0,d1,d2,d3}, {%10,%11,%12,%13}, {%22,%23}, {d0,d1,d2,d3};\n\t"
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {d0,d1,d2,d3}, {%14,%15,%16,%17}, {%24,%25}, {d0,d1,d2,d3};\n\t"
        "mov.b64 %0, {d0,d1};\n\t"
        "mov.b64 %1, {d2,d3};\n\t}"
        : "=l"(lo), "=l"(hi)
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(a[4]), "r"(a[5]), "r"(a[6]), "r"(a[7]), "r"(a[8]), "r"(a[9]), "r"(a[10]), "r"(a[11]),
          "r"(a[12]), "r"(a[13]), "r"(a[14]), "r"(a[15]), "r"(b[0]), "r"(b[1]), "r"(b[2]), "r"(b[3]), "r"(b[4]), "r"(b[5]), "r"(b[6]), "r"(b[7]),
          "r"(c));
}

// A 16-byte load from shared memory that only the lanes with `on` perform; the others keep what
// `v` held (a predicated instruction: lanes that are off cost no shared-memory bandwidth).
__device__ __forceinline__ void lds128_if(uint4& v, uint32_t addr, bool on) {   // addr: smem_u32() of the source
    asm volatile(
        "{\n\t.reg .pred q;\n\t"
        "setp.ne.u32 q, %4, 0;\n\t"
        "@q ld.shared.v4.u32 {%0,%1,%2,%3}, [%5];\n\t}"
        : "+r"(v.x), "+r"(v.y), "+r"(v.z), "+r"(v.w)
        : "r"(uint32_t(on)), "r"(addr));
}

__device__ __forceinline__ void mma_u8s8_bias(uint64_t& lo, uint64_t& hi, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                              uint32_t b0, uint32_t b1, int c) {
    asm volatile(
        "{\n\t.reg .b32 d0, d1, d2, d3;\n\t"
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {d0,d1,d2,d3}, {%2,%3,%4,%5}, {%6,%7}, {%8,%8,%8,%8};\n\t"
        "mov.b64 %0, {d0,d1};\n\t"
        "mov.b64 %1, {d2,d3};\n\t}"
        : "=l"(lo), "=l"(hi)
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(c));
}

// Packed fp32 pairs (sm_100 f32x2 arithmetic): each half is an IEEE round-to-nearest operation,
// so results are the same as two scalar instructions at half the issue slots. One caveat, seen on
// B200: a packed multiply whose result feeds a packed add is contracted into a packed fused
// multiply-add, even with .rn on both; where the two roundings matter, do one of the two scalar.
__device__ __forceinline__ uint64_t pack2(float a, float b) {
    uint64_t r;
    asm("mov.b64 %0, {%1,%2};" : "=l"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& a, float& b) { asm("mov.b64 {%0,%1}, %2;" : "=f"(a), "=f"(b) : "l"(v)); }
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ uint64_t sub2(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}

// ---- oracle-exact scalar pieces (no FMA contraction, IEEE division; never built with fast-math)

// roundf: to nearest, halves away from zero
__device__ __forceinline__ float round_half_away(float v) {
    const float t = truncf(v);
    const float f = __fsub_rn(v, t);   // exact
    return fabsf(f) >= 0.5f ? t + copysignf(1.0f, v) : t;
}

// Correctly rounded expf for all but a vanishing fraction of inputs: exp in double to about 2^-51,
// then one rounding to float. e^x = 2^k * e^r with k = round(x / ln 2) and r = x - k ln 2
// (ln 2 as a 32-bit head, so that k * head is exact, and a tail), |r| <= 0.347, e^r by its Taylor
// series to r^13 / 13! (the next term is below 2^-57). Half the double-precision work of the
// library's exp, which matters where this sits at the end of a tile. Identical to
// float(exp(double(x))) on 5e7 random inputs checked on the host.
__device__ __forceinline__ float expf_cr(float x) {
    if (!(x == x)) return x;
    const double xd = double(fminf(fmaxf(x, -110.0f), 90.0f));   // beyond: 0 or inf as a float either way
    const double kd = rint(xd * 1.4426950408889634);
    double r = fma(-kd, 0x1.62e42fee00000p-1, xd);
    r = fma(-kd, 0x1.a39ef35793c76p-33, r);
    double p = 1.0 / 6227020800.0;
    p = fma(p, r, 1.0 / 479001600.0);
    p = fma(p, r, 1.0 / 39916800.0);
    p = fma(p, r, 1.0 / 3628800.0);
    p = fma(p, r, 1.0 / 362880.0);
    p = fma(p, r, 1.0 / 40320.0);
    p = fma(p, r, 1.0 / 5040.0);
    p = fma(p, r, 1.0 / 720.0);
    p = fma(p, r, 1.0 / 120.0);
    p = fma(p, r, 1.0 / 24.0);
    p = fma(p, r, 1.0 / 6.0);
    p = fma(p, r, 0.5);
    p = fma(p, r, 1.0);
    p = fma(p, r, 1.0);
    const double scale = __hiloint2double((__double2int_rn(kd) + 1023) << 20, 0);   // 2^k, k in [-159, 130]
    return __double2float_rn(p * scale);
}

// silu(g) * u as the reference's CPU path writes it: g / (1 + exp(-g)) * u
__device__ __forceinline__ float swiglu_ref(float g, float u) {
    const float e = expf_cr(-g);
    return __fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, e)), u);
}

__device__ __forceinline__ float sigmoid_ref(float x) { return __fdiv_rn(1.0f, __fadd_rn(1.0f, expf_cr(-x))); }

}  // namespace frx
