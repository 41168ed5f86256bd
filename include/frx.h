/*
 * libfrx: the Q2_0 MoE expert path of flashrt on B200 (sm_100a), as a C ABI over CUDA.
 *
 * The reference has no plugin or FFI layer: the path is reached through C++ free functions that
 * its MoE blocks call (moe_q2::run, qwen4exp::moe_route_topk, qwen4exp::moe_hits, the combine
 * kernels). Every entry point here names the reference interface it stands in for; frx_shim.hpp
 * re-declares those functions with the reference's own signatures on top of this header.
 *
 * Conventions (the reference's, arch/qwen4exp/blocks.hpp and kernels/cuda/moe_q2.h):
 *   - every pointer is a device pointer unless its name ends in _host;
 *   - row-major, token-major layouts; the caller owns inputs, outputs and workspaces and asks
 *     the *_bytes functions for sizes; nothing is allocated by a compute call;
 *   - activation and output buffers ([T][n] float rows, per-slot rows) are 16-byte aligned, int8
 *     code buffers 4-byte aligned (n is a multiple of 128, so every row is when the base is);
 *     a misaligned pointer is refused with FRX_ERR_ARG;
 *   - work is enqueued on the caller's stream, with no host synchronisation;
 *   - a call returns FRX_OK or an error code and never throws; frx_last_error() gives the text
 *     of the calling thread's last error.
 *
 * Expert weights are Q2_0 (ggml type 42): blocks of 64 weights, one fp16 scale d and 64 two-bit
 * codes q, a weight being (q - 1) * d. Compute entry points take experts in the *tiled* layout
 * described at frx_q2_tile_experts, which holds the same 18 bytes per block as the reference's
 * planar layout, reordered.
 *
 * Numerics: activations are quantized to int8 per 32 values exactly as the reference's CPU path
 * does (quant/q2_0/q2_0.cpp:101-113), the integer dot products are exact, and the float scaling
 * and summation follow the order of the reference's scalar matvec (quant/q2_0/q2_0.cpp:119-140).
 */
#ifndef FRX_H
#define FRX_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* frx_stream_t; /* a cudaStream_t */

enum {
    FRX_OK = 0,
    FRX_ERR_ARG = 1,       /* null pointer, negative size, misaligned pointer */
    FRX_ERR_SHAPE = 2,     /* a shape the kernels do not support */
    FRX_ERR_WORKSPACE = 3, /* workspace smaller than *_workspace_bytes says */
    FRX_ERR_CUDA = 4,      /* a CUDA runtime call or launch failed */
    FRX_ERR_DEVICE = 5     /* a kernel reported an error (bad expert id, a wait that ran out) */
};

int frx_version(void);
const char* frx_last_error(void);

/* Per-kernel timing for benchmarks; no counterpart in the reference (it profiles with nsys).
 * Between frx_profile_begin() and frx_profile_end(), every kernel the library launches is bracketed
 * by two CUDA events on its stream. frx_profile_end waits for them and returns, per kernel class c
 * (frx_profile_class_name(c): "route_topk", "quant_q8", "group", "gate_up", "down", "combine",
 * "layout"), the summed device time ms[c] and the launch count launches[c]. Not for use while a
 * stream is being captured into a CUDA graph. */
int frx_profile_begin(void);
int frx_profile_end(float* ms, int* launches, int n_classes);
const char* frx_profile_class_name(int cls);

/* Tuning knobs for measurements and tests; no counterpart in the reference. Process-wide and not
 * thread-safe: set them before any compute call, not while calls are in flight.
 * frx_debug_set_consumer_warps: warps per block of the streaming expert kernel (8, 12, 16 or 20; default 16).
 * frx_debug_set_gate_up_chunks: the number of K slices a gate/up task is fetched in (0: chosen by shape).
 * frx_debug_set_narrow_items: 1 (default) lets work items of at most four tokens take the narrow
 * form of the inner product (two row groups share one MMA accumulator, half the float work per row);
 * 0 sends every item through the eight-token form. Results are the same bits either way.
 * frx_debug_set_fused_ffn: 1 runs the expert FFN of the decode layer (gate/up, the hidden rows, down) as one
 * kernel when items have at most four tokens and the shape allows; 0 (default, the faster as measured) keeps
 * the three kernels. frx_debug_set_ffn_buffers: item buffers per half of that kernel (0 = as many as fit,
 * at most three). Same bits either way.
 * frx_debug_set_four_group_tasks: which streaming kernels of the decode layer walk four row groups per task
 * instead of two (needs narrow items): bit 0 gate/up, bit 1 down; default 2 (down only, the faster
 * combination as measured). Same bits either way.
 * frx_debug_set_wait_limit_ns: the longest a kernel waits on a barrier, a flag or a peer before it
 * gives up and reports FRX_ERR_DEVICE through the workspace status (default 2 s; 0 restores it). */
int frx_debug_set_consumer_warps(int nw);
/* Launches with at most `four_warps` (`eight_warps`) tasks per SM use blocks of 4 (8) warps with deeper copy rings
 * instead of the setting above (defaults 0 and 8; 0, 0: never). */
int frx_debug_set_small_launch_limits(int four_warps, int eight_warps);
int frx_debug_set_gate_up_chunks(int chunks);
int frx_debug_set_narrow_items(int on);
int frx_debug_set_four_group_tasks(int on);
int frx_debug_set_fused_ffn(int on);
/* 1 (default): in the decode layer the down kernel forms and quantizes the hidden rows while it builds its
 * item buffers (needs narrow items and four-group tasks in down); 0: a separate quantizer kernel writes them
 * to the workspace first (where frx_decode_workspace_view can read them). Same bits either way. */
int frx_debug_set_fold_quant(int on);
/* 1 (default): the decode layer's weight copies mark their L2 lines evict-first (a layer's 326 MB of experts pass
 * once through a 126 MB L2 and would otherwise push out the kernels' code and the small buffers that are read
 * again); 0: default policy. */
int frx_debug_set_evict_first(int on);
/* Decode layer: the down kernel's tasks are shared out among its blocks by weight, a task of an item of three
 * or four tokens weighing `sixteenths` / 16 of one of a smaller item (default 22; 16 = equal; 0 = an even
 * split by count, made by the kernel itself). Same bits whatever the split. */
int frx_debug_set_down_task_weight(int sixteenths);
/* ... and every item weighs `sixteenths` / 16 tasks more (its item buffer, built by every block that has tasks
 * of it); default 256. */
int frx_debug_set_down_item_weight(int sixteenths);
/* Measurement aid: with a device buffer of (2 * SMs + 1) * 4 * 8 bytes set, every launch of the decode layer's two
 * streaming kernels (three-kernel form) writes four globaltimer stamps per block there, gate/up's blocks first,
 * then down's: [0] block started, [1] the kernels in front have ended, [2] first item buffer built, [3] block
 * finished; and block 0 of the layer's first kernel four more behind them: [0] the kernels in front have ended,
 * [1] its own tokens routed, [2] all tokens routed, [3] work items written. NULL (default) switches it off. */
int frx_debug_set_stream_stamps(void* device_buffer);
int frx_debug_set_ffn_buffers(int gate_up, int down);
int frx_debug_set_wait_limit_ns(unsigned long long ns);

/* ---- Q2_0 storage (quant/q2_0/q2_0.hpp:27-56, quant/q2_0/q2_0.cpp:43-71) ---- */

/* q2_0::mat_bytes, q2_0::expert_bytes: rows * (cols / 64) * 18; gate + up + down. */
size_t frx_q2_mat_bytes(int rows, int cols);
size_t frx_q2_expert_bytes(int n, int ff);
/* ExpertArena's stride rule (core/expert_arena.hpp:14-24): the blob rounded up to 4 KiB. */
size_t frx_q2_expert_stride(int n, int ff);

/* q2_0::repack (quant/q2_0/q2_0.cpp:51-62) on the device: `rows` rows of ggml blocks
 * {fp16 d; 16 code bytes, element j in byte j/4 at bit 2*(j%4)} to the planar layout
 * (codes [rows][cols/64][16], element j in byte j%16 at bit 2*(j/16); then scales [rows][cols/64]). */
int frx_q2_repack(const void* ggml_rows, int rows, int cols, void* planar, frx_stream_t stream);

/* Planar expert blobs (q2_0::expert_view: gate [ff][n], up [ff][n], down [n][ff]) to the tiled
 * layout the kernels read, and back. Needs n % 128 == 0, ff % 128 == 0. Blob e is read at
 * src + e * src_stride and written at dst + e * dst_stride; both hold frx_q2_expert_bytes(n, ff).
 *
 * Tiled layout. A *unit* is 16 matrix rows ("M rows") by 2 blocks (128 weights of K), 576 bytes:
 *   bytes [0, 512): for lane L = 0..31 (g = L >> 2, t = L & 3) four 32-bit words [h][j],
 *                   h, j in {0, 1}: bytes 4t..4t+3 of the planar 16-byte block of M row g + 8h,
 *                   block 2u + j (so field p of byte i holds element 16p + 4t + i of the block);
 *   bytes [512, 576): fp16 scales [g][h][j] of the same blocks.
 * A *group* is the units u = 0..K/128-1 of 16 M rows, back to back. The blob is
 *   gate/up groups G = 0..ff/8-1: M row m < 8 is gate row 8G + m, M row 8 + m is up row 8G + m,
 *                                  K = n;
 *   down groups G = 0..n/16-1:    M row m is down row 16G + m, K = ff.
 * One lane's 16-byte load of a unit yields the int8 MMA A fragments of two blocks by shifts and a
 * mask; a group is one contiguous, 64-byte-aligned stream for a bulk copy. */
int frx_q2_tile_experts(const void* src_planar, size_t src_stride, void* dst_tiled, size_t dst_stride, int n_experts,
                        int n, int ff, frx_stream_t stream);
int frx_q2_untile_experts(const void* src_tiled, size_t src_stride, void* dst_planar, size_t dst_stride, int n_experts,
                          int n, int ff, frx_stream_t stream);

/* Dequantised weights (q - 1) * float(d) of one tiled expert: gate, up [ff][n], down [n][ff]
 * fp32 (any of the three may be null). The values the reference's tests compute element by
 * element (tests/test_q2_0.cpp:56-60). */
int frx_q2_dequant_expert(const void* tiled_blob, int n, int ff, float* gate, float* up, float* down,
                          frx_stream_t stream);

/* ---- HBM-resident expert arena (replaces core/expert_arena.hpp:14-30, which is host memory) ---- */

typedef struct frx_arena frx_arena;
/* One device allocation of n_layer * n_expert tiled blobs, blob (l, e) at
 * base + (l * n_expert + e) * stride, stride = frx_q2_expert_stride(n, ff). */
int frx_arena_create(frx_arena** out, int n_layer, int n_expert, int n, int ff);
int frx_arena_destroy(frx_arena* a);
void* frx_arena_base(const frx_arena* a);
void* frx_arena_blob(const frx_arena* a, int layer, int expert); /* ExpertArena::blob */
size_t frx_arena_stride(const frx_arena* a);
size_t frx_arena_total_bytes(const frx_arena* a);
/* Copies `count` planar blobs (host or device memory, src_stride apart) into blobs
 * (layer, expert0 ..) of the arena, converting them to the tiled layout on the way. */
int frx_arena_load_planar(frx_arena* a, int layer, int expert0, int count, const void* src_planar, size_t src_stride,
                          frx_stream_t stream);

/* ---- routing: qwen4exp::moe_route_topk (arch/qwen4exp/blocks.hpp:134-135, moe_ref.cu:21-86) ----
 * Softmax over E <= 1024 logits per token, the k <= 32 most probable experts in descending
 * probability with ties to the lower index, weights p / max(sum of the selected p, 6.103515625e-5).
 * ids, wts [T][k]. counts [E] (may be null): each selection adds 1. tail_counts [E] (may be null):
 * rows t >= tail_from also add 1 there.
 * The ranking is done on the logits (the softmax is monotonic; -0.0 and +0.0 tie). One corner differs
 * from the reference, which ranks on the float probabilities: two distinct logits whose probabilities
 * round to the same float, or both underflow to zero (a logit more than about 103 below the row's
 * maximum), tie there and go to the lower index, while here the larger logit wins. */
int frx_route_topk(frx_stream_t stream, const float* logits, int T, int E, int k, int32_t* ids, float* wts,
                   uint32_t* counts, uint32_t* tail_counts, int tail_from);

/* ---- activation quantizer: q2_0::quantize_q8 (quant/q2_0/q2_0.cpp:101-117) ----
 * Per 32 values: d = amax / 127, q = roundf(x / d) (half away from zero), d stored after a
 * round trip through fp16. x [T][n]; q [T][n] int8; d [T][n/32] float. n % 32 == 0. */
int frx_quantize_q8(frx_stream_t stream, const float* x, int T, int n, int8_t* q, float* d);

/* ---- decode-sized MoE layer (T tokens, any T; tuned for T <= 64) ----
 * Stands in for the MoE block of a decode step (arch/qwen4exp/moe_fast.cu:1015-1108 and
 * arch/qwen4exp/moe_ref.cu:106-190) with every expert resident in device memory:
 *   out[t] = sum over the token's K experts, in ascending expert id, of wts * expert(x_t)
 *            (the accumulation order of quant/q2_0/moe_cpu.cpp:70-79)
 *          + shared(x_t) * sigmoid(gate_logit[t])        (moe_ref.cu:91-97), if shared != null.
 * experts: tiled blobs at experts + e * stride, e < E. shared: one tiled blob or null.
 * gate_logit [T] or null (weight 1). ids, wts [T][K] as frx_route_topk writes them.
 * yslot (may be null): per-slot expert outputs [T*K][n], slot t*K+k, the moe_q2::run / moe_hits
 * output contract. n % 128 == 0, ff % 128 == 0, K <= 32, n <= 8192, ff <= 8192; out and yslot
 * 16-byte aligned. */
size_t frx_moe_decode_workspace_bytes(int T, int K, int n, int ff);
int frx_moe_decode(const void* experts, size_t stride, int E, const void* shared, int n, int ff, const float* x,
                   const int32_t* ids, const float* wts, const float* gate_logit, int T, int K, float* out, float* yslot,
                   void* ws, size_t ws_bytes, frx_stream_t stream);

/* Expert-parallel form; no counterpart in the reference, which runs on one GPU. This rank holds
 * the experts [e_lo, e_hi) of E, expert e at experts + (e - e_lo) * stride; ids still name experts
 * in [0, E). out[t] is the partial sum over the token's slots whose expert lives here (plus the
 * shared term if shared != null: give the shared expert to one rank only); the sum of the ranks'
 * outputs is the layer output. yslot rows of experts held elsewhere are not written. */
int frx_moe_decode_ep(const void* experts, size_t stride, int E, int e_lo, int e_hi, const void* shared, int n, int ff,
                      const float* x, const int32_t* ids, const float* wts, const float* gate_logit, int T, int K, float* out,
                      float* yslot, void* ws, size_t ws_bytes, frx_stream_t stream);

/* frx_moe_decode without a caller-supplied workspace, for hosts that cannot allocate device memory
 * once they are running (an engine that gave all free device memory to its caches at start-up, a
 * loop that must not call cudaMalloc after initialisation, a plugin host that owns the allocator).
 * It has no counterpart in the reference. The scratch is a fixed 4 MiB array inside the library's
 * device image (held by every GPU that loads the library, until the process exits); the call
 * allocates and frees nothing. Same arguments and result as frx_moe_decode with yslot = null.
 * Limits and rules:
 *   - T, K, n, ff must satisfy frx_moe_decode_workspace_bytes(T, K, n, ff) <= 4 MiB (for n = 2048,
 *     ff = 512, K = 10 that is up to 24 tokens); otherwise FRX_ERR_WORKSPACE, and the message
 *     gives both sizes;
 *   - the first call on each device looks up the array's device address (with that device
 *     current); make that first call before any stream capture begins;
 *   - all calls on a device share the one array: calls whose kernels can overlap on the GPU (two
 *     streams, two host threads) race on it, so keep them on one stream or order them;
 *   - a kernel error (a bad expert id, a bounded wait that ran out) is flagged in the scratch;
 *     frx_moe_decode_static_status reads and clears it (it synchronises the stream, allocates nothing). */
int frx_moe_decode_static(const void* experts, size_t stride, int E, const void* shared, int n, int ff, const float* x,
                          const int32_t* ids, const float* wts, const float* gate_logit, int T, int K, float* out,
                          frx_stream_t stream);
int frx_moe_decode_static_status(frx_stream_t stream);

/* Byte offset, inside a frx_moe_decode workspace, of one of its buffers (for tests and debugging).
 * "xq" int8 [T][n], "xa" float [T][n/32], "xc" float [T][n/32]: the Q8 form of x as the expert
 * kernel reads it -- the four codes of elements 64b + 32s + 16h + 4t .. +3 of a row are word
 * (b*4 + t)*4 + s*2 + h; xa is the block scale, divided by 16 for odd blocks; xc is
 * 12582912 + sum(codes) as a float, the sum times 16 for odd blocks. "hq", "ha", "hc": the same for the
 * hidden activations, one row of ff per slot. "h" float [T*K + T][ff]: the hidden activations
 * silu(gate x) * up x per slot (shared-expert slots last). "y" float [T*K][n], "ysh" float [T][n],
 * "order" int32 [T][K]. Valid for T <= 64. Returns (size_t)-1 for other names. */
size_t frx_moe_decode_workspace_offset(int T, int K, int n, int ff, const char* what);

/* ---- GGUF container and the expert loader (core/gguf.hpp:17-60, arch/qwen4exp/experts.cpp:65-131) ----
 * frx_gguf_open parses the metadata and the tensor directory of one GGUF file (format version 2 or
 * 3; split files are not handled); tensor data stays on disk. frx_gguf_tensor reports a tensor's
 * ggml type id, dimensions (fastest first, unused ones 1), absolute file offset and byte count.
 * frx_arena_load_gguf reads the Q2_0 expert tensors blk.<l>.ffn_{gate,up,down}_exps.weight (ggml type
 * 42, expert e's matrix at e * mat_bytes) of layers [layer0, layer0 + n_layer) and fills arena
 * layers of the same numbers: repacked to the planar form and tiled on the device. It allocates
 * its staging (pinned host and device) for the duration of the call and returns after the stream
 * has drained; bytes_read / seconds (may be null) report the volume and the wall time. */
typedef struct frx_gguf frx_gguf;
int frx_gguf_open(frx_gguf** out, const char* path);
int frx_gguf_close(frx_gguf* g);
int frx_gguf_tensor_count(const frx_gguf* g);
const char* frx_gguf_tensor_name(const frx_gguf* g, int i);
int64_t frx_gguf_get_int(const frx_gguf* g, const char* key, int64_t fallback);   /* integer or boolean metadata */
int frx_gguf_tensor(const frx_gguf* g, const char* name, uint32_t* type, int* n_dims, int64_t* dims4, uint64_t* file_offset,
                    uint64_t* bytes);
int frx_arena_load_gguf(frx_arena* a, const frx_gguf* g, int layer0, int n_layer, int n_expert, int n, int ff, frx_stream_t stream,
                        uint64_t* bytes_read, double* seconds);

/* The projection in front of the router (k_bf16_multi, arch/qwen4exp/blocks.cu:83-120, as called at
 * moe_fast.cu:1039-1042 and moe_stream.cu:145-149): logits[t][e] = sum_k w_router[e][k] * x[t][k],
 * w_router bf16 [E][n] row-major, x fp32 [T][n], exact products and fp32 sums; with w_gate (bf16 [n],
 * may be null) also gate_logit[t] = sum_k w_gate[k] * x[t][k], the shared expert's gate logit that
 * frx_moe_layer takes. n a multiple of 256 (as in the reference), pointers 16-byte aligned. */
int frx_router_logits(frx_stream_t stream, const void* w_router, const void* w_gate, const float* x, int T, int E, int n,
                      float* logits, float* gate_logit);

/* Router + layer in one call: logits [T][E] -> top-K -> frx_moe_decode. ids_out / wts_out [T][K]
 * (may be null) receive the routing. Workspace: frx_moe_layer_workspace_bytes. */
size_t frx_moe_layer_workspace_bytes(int T, int K, int n, int ff);
int frx_moe_layer(const void* experts, size_t stride, int E, const void* shared, int n, int ff, const float* x,
                  const float* logits, const float* gate_logit, int T, int K, float* out, int32_t* ids_out,
                  float* wts_out, void* ws, size_t ws_bytes, frx_stream_t stream);

/* Expert-parallel form of frx_moe_layer: every rank routes (the logits are replicated, so ids and
 * weights are identical everywhere), this rank computes the experts [e_lo, e_hi) it holds
 * (`experts_local` points at the blob of expert e_lo) and `out` receives its partial sums, as
 * frx_moe_decode_ep. */
int frx_moe_layer_ep(const void* experts_local, size_t stride, int E, int e_lo, int e_hi, const void* shared, int n, int ff,
                     const float* x, const float* logits, const float* gate_logit, int T, int K, float* out, int32_t* ids_out,
                     float* wts_out, void* ws, size_t ws_bytes, frx_stream_t stream);

/* ---- Expert parallel with the all-reduce fused into the combine (peer memory over NVLink) ------
 *
 * Every rank owns one communication buffer (frx_ep_buffer_create; device memory that other
 * processes of the node map through CUDA IPC: frx_ipc_export / frx_ipc_open). It holds two slots of
 * partial sums [max_T][n] fp32, one flag word per peer and block, and a few local counters. frx_ep_comm lists
 * every rank's buffer as mapped on this device (entry `rank` is the local one).
 *
 * frx_moe_layer_ep_allreduce = frx_moe_layer_ep, but its last kernel, after forming this rank's
 * weighted partial sums, stores them into the rank's own buffer, tells every peer (one flag word
 * per block, release at system scope), waits until every peer has told it (bounded: after 2 s, or
 * the limit set with frx_debug_set_wait_limit_ns, the workspace status reports a time-out and the
 * kernel finishes without hanging), and adds the peers' partial sums
 * to its own, in rank order on every rank, so all ranks get the same bits. `out` then holds the
 * complete layer output on every rank. No NCCL call is involved, so a step can be captured in a
 * CUDA graph. All ranks must make the same sequence of calls with the same comm; T <= 64 and
 * T <= max_T. The reference is single-GPU and has no counterpart. */
#define FRX_EP_MAX_RANKS 8
typedef struct frx_ep_comm {
    int world, rank;
    int max_T, n;
    void* buffer[FRX_EP_MAX_RANKS]; /* every rank's communication buffer, as mapped on this device */
} frx_ep_comm;
#define FRX_EP_MAX_BLOCKS 1024
size_t frx_ep_buffer_bytes(int max_T, int n);
/* Byte offset of the flag words inside a buffer: uint32 [FRX_EP_MAX_RANKS][FRX_EP_MAX_BLOCKS], word
 * [q][b] = number of the last call whose partial sums block b of rank q has published here. The two
 * slots of partial sums (slot = call number & 1, calls counted from 1) start at offset 0 and
 * max_T * n * 4. For tests and debugging. */
size_t frx_ep_flags_offset(int max_T, int n);
int frx_ep_buffer_create(void** buffer, int max_T, int n);   /* allocated and zeroed; once, at set-up */
int frx_ep_buffer_destroy(void* buffer);
#define FRX_IPC_HANDLE_BYTES 64
int frx_ipc_export(const void* buffer, void* handle);        /* handle: FRX_IPC_HANDLE_BYTES bytes to send to the peers */
int frx_ipc_open(const void* handle, void** mapped);         /* a peer's buffer on this device */
int frx_ipc_close(void* mapped);
/* Tear-down order: a buffer may be destroyed only after every rank has finished its last call that
 * uses it (device synchronised) and every peer has closed its mapping of it; a peer's last kernel
 * may otherwise still be reading it over NVLink. */
/* Measurement aid: SM cycle stamps (clock64 of block 0) of the last frx_moe_layer_ep_allreduce call
 * on this rank: [0] kernel start, [1] partial sums stored, [2] every peer's flag seen, [3] peers'
 * parts read and summed. own_buffer is this rank's buffer; the call copies synchronously. */
int frx_ep_debug_stamps(const void* own_buffer, int max_T, int n, long long* cycles4);
int frx_moe_layer_ep_allreduce(const void* experts_local, size_t stride, int E, int e_lo, int e_hi, const void* shared, int n, int ff,
                               const float* x, const float* logits, const float* gate_logit, int T, int K, float* out,
                               int32_t* ids_out, float* wts_out, const frx_ep_comm* comm, void* ws, size_t ws_bytes,
                               frx_stream_t stream);

/* The same with the shared expert's work dealt among the ranks: every rank holds a copy of the shared
 * expert and applies it to the tokens [shared_t0, shared_t1) (an empty range: none); the ranges of the
 * ranks must partition [0, T). With the plain entry the one rank that passes `shared` does all T
 * tokens and is the last to arrive at every exchange. Ranges that are multiples of four tokens keep
 * the work items full. */
int frx_moe_layer_ep_allreduce_dealt(const void* experts_local, size_t stride, int E, int e_lo, int e_hi, const void* shared,
                                     int shared_t0, int shared_t1, int n, int ff, const float* x, const float* logits,
                                     const float* gate_logit, int T, int K, float* out, int32_t* ids_out, float* wts_out,
                                     const frx_ep_comm* comm, void* ws, size_t ws_bytes, frx_stream_t stream);

/* The same with host buffers: x_host [T][n], logits_host [T][E], gate_logit_host [T] or null are
 * copied to the device, the layer runs, out_host [T][n] is copied back, and the call returns after
 * the stream has drained. `ws` is a device workspace of frx_moe_layer_host_workspace_bytes. */
size_t frx_moe_layer_host_workspace_bytes(int T, int K, int n, int ff, int E);
int frx_moe_layer_host(const void* experts, size_t stride, int E, const void* shared, int n, int ff,
                       const float* x_host, const float* logits_host, const float* gate_logit_host, int T, int K,
                       float* out_host, void* ws, size_t ws_bytes, frx_stream_t stream);

/* L independent layer calls from host buffers in one call, pipelined: while layer l computes on
 * `stream`, the inputs of the following layers are copied in and the outputs of the preceding ones
 * copied out on two copy streams the library creates once per device (at the first call; call it
 * once outside any stream capture). experts[l], shared[l] (shared may be null, or shared[l] null):
 * device blobs of layer l; x_host[l] [T][n], logits_host[l] [T][E], gate_logit_host[l] [T] (the
 * array or an entry may be null), out_host[l] [T][n]: host buffers, pinned if the copies are to
 * overlap. Calls on one device must not run concurrently (they share the copy streams and their
 * events). Results are bit-identical to L calls of frx_moe_layer_host. Returns after everything
 * has drained. `ws`: device workspace of frx_moe_layers_host_workspace_bytes (independent of L:
 * inputs and outputs pass through a ring of four staging slots). The reference has no counterpart:
 * its engine keeps activations on the device between layers. */
size_t frx_moe_layers_host_workspace_bytes(int T, int K, int n, int ff, int E);
int frx_moe_layers_host(const void* const* experts, size_t stride, int E, const void* const* shared, int n, int ff,
                        const float* const* x_host, const float* const* logits_host, const float* const* gate_logit_host,
                        int L, int T, int K, float* const* out_host, void* ws, size_t ws_bytes, frx_stream_t stream);

/* Waits for the stream, then: FRX_OK, or FRX_ERR_DEVICE if a kernel of a call that used this
 * workspace reported an error (then frx_last_error() says which: an expert id out of range, more
 * work items than the workspace holds, or a bounded wait that ran out). An error is reported once:
 * the call clears it, so later calls on the same workspace start clean. */
int frx_workspace_status(const void* ws, frx_stream_t stream);

/* ---- qwen4exp::moe_hits (arch/qwen4exp/moe_fast.hpp:134-142) ----
 * yh[t][k] [n] = down_k(silu(gate_k x_t) * up_k x_t) for k < hit_n[t], expert k's tiled blob at
 * hit_ptr[t*K + k] (device array of device pointers); rows k >= hit_n[t] are not written. An
 * expert that several tokens of the window hit is read once. x [T][n]; yh [T][K][n]. T*K <= 1024.
 * Unlike the reference's kernel, activations are quantized per 32 with round-half-away, which is
 * what the reference's CPU path does. */
size_t frx_moe_hits_scratch_bytes(int K, int n, int ff, int T);
int frx_moe_hits(const uint8_t* const* hit_ptr, const int32_t* hit_n, int K, const float* x, int n, int ff, void* scratch,
                 size_t scratch_bytes, float* yh, frx_stream_t stream, int T);

/* ---- combine: k_moe_combine (arch/qwen4exp/moe_fast.cu:499-508), k_stream_combine
 * (arch/qwen4exp/moe_stream.cu:40-46) ----
 * out[t] = sum_{k < hit_n[t]} w[t][k] * yh[t][k] (in k order) + shexp[t] * sigmoid(gate[t]).
 * hit_n null means K for every token; shexp / gate null drop the shared term / use weight 1. */
int frx_moe_combine(float* out, const float* yh, const float* w, const int32_t* hit_n, const float* shexp,
                    const float* gate, int n, int K, int T, frx_stream_t stream);

/* ---- prefill-sized grouped expert product: moe_q2::run (kernels/cuda/moe_q2.h:21-30) ----
 * yd[t*K + k] [n] = down(silu(gate x_t) * up x_t) of expert ids[t*K + k], fp32.
 * Grouping by expert, the tile list and every launch size are computed on the device: no host
 * synchronisation. n % 128 == 0, ff % 128 == 0, E <= 4096.
 * Two forms compute the same bits: frx_moe_prefill_umma runs the integer products on the tcgen05
 * tensor cores with accumulators in tensor memory, frx_moe_prefill_stream is the form the decode
 * path uses. frx_moe_prefill takes the tensor-memory form when experts receive 256 or more tokens
 * on average (T * K >= 256 * E) and the streaming form otherwise; the two are exported so each can
 * be called and measured on its own, with the same arguments and workspace size. */
size_t frx_moe_prefill_workspace_bytes(int T, int K, int n, int ff, int E);
int frx_moe_prefill(const void* experts, size_t stride, int E, int n, int ff, const float* x, const int32_t* ids, int T,
                    int K, float* yd, void* ws, size_t ws_bytes, frx_stream_t stream);
int frx_moe_prefill_umma(const void* experts, size_t stride, int E, int n, int ff, const float* x, const int32_t* ids, int T,
                         int K, float* yd, void* ws, size_t ws_bytes, frx_stream_t stream);
int frx_moe_prefill_stream(const void* experts, size_t stride, int E, int n, int ff, const float* x, const int32_t* ids, int T,
                           int K, float* yd, void* ws, size_t ws_bytes, frx_stream_t stream);
/* The same with moe_q2::run's two options (kernels/cuda/moe_q2.h:26-30). block64: activations (x and
 * the hidden rows) are quantized with one scale per 64 values instead of per 32 (the scale still
 * passes through fp16 and codes round half away from zero; the reference's CPU path has no such
 * mode, so this one is checked against it within the reference test's own bound,
 * tests/test_moe_q2.cpp:139-141). yd_bf16: yd receives bf16 rows [T*K][n] (round to nearest) as
 * arch/qwen4exp/moe_stream.cu:164-177 wants them. */
int frx_moe_prefill_ex(const void* experts, size_t stride, int E, int n, int ff, const float* x, const int32_t* ids, int T,
                       int K, void* yd, void* ws, size_t ws_bytes, frx_stream_t stream, int block64, int yd_bf16);
int frx_moe_prefill_umma_ex(const void* experts, size_t stride, int E, int n, int ff, const float* x, const int32_t* ids, int T,
                            int K, void* yd, void* ws, size_t ws_bytes, frx_stream_t stream, int block64, int yd_bf16);
int frx_moe_prefill_stream_ex(const void* experts, size_t stride, int E, int n, int ff, const float* x, const int32_t* ids, int T,
                              int K, void* yd, void* ws, size_t ws_bytes, frx_stream_t stream, int block64, int yd_bf16);

/* ---- expert-parallel prefill (tokens and experts both sharded over the GPUs of a node; the
 * reference runs on one GPU and has no counterpart; the nearest single-GPU structure is
 * arch/qwen4exp/moe_stream.cu:152-177) ----
 * Every rank quantizes its own tokens (frx_quantize_q8: 2,304 bytes per token instead of 8,192),
 * the ranks exchange the quantized tokens and the routing (all-gather), each rank runs
 * frx_moe_prefill_q8_ep over all T tokens but only over the slots whose expert it holds, forms its
 * part of every token's weighted sum (frx_moe_combine_partial), and a reduce-scatter of those rows
 * gives every rank the outputs of its own tokens. Nothing here waits for the stream.
 * e_map [E_all] int32 (device): the index of every expert among the E_local held by this rank
 * (experts_local + index * stride), or -1: any placement of experts on ranks, e.g. hot experts
 * dealt round-robin. xq [T][n] int8 and xd [T][n/32] float as frx_quantize_q8 writes them; ids [T][K]
 * name experts of the whole layer. yd [T*K][n]: rows of slots held elsewhere are not written.
 * form: 0 by size, 1 streaming, 2 tensor-memory. Workspace: frx_moe_prefill_workspace_bytes(T, K, n, ff, E_local). */
int frx_moe_prefill_q8_ep(const void* experts_local, size_t stride, int E_local, const int32_t* e_map, int E_all, int n, int ff,
                          const int8_t* xq, const float* xd, const int32_t* ids, int T, int K, float* yd, void* ws, size_t ws_bytes,
                          frx_stream_t stream, int form);
/* The streaming form of frx_moe_prefill_q8_ep on its own (form = 1). */
int frx_moe_prefill_stream_q8_ep(const void* experts_local, size_t stride, int E_local, const int32_t* e_map, int E_all, int n, int ff,
                                 const int8_t* xq, const float* xd, const int32_t* ids, int T, int K, float* yd, void* ws, size_t ws_bytes,
                                 frx_stream_t stream);
/* out[t] = sum over the token's slots whose expert is held here (e_map[id] >= 0), in ascending
 * expert id, of wts * yd; zeros for tokens with no such slot. out [T][n]. */
int frx_moe_combine_partial(float* out, const float* yd, const float* wts, const int32_t* ids, const int32_t* e_map, int n, int K, int T,
                            frx_stream_t stream);

/* The join between layers of the chained expert-stack benchmark (a 48-layer stack walked by a
 * window of three tokens): x_next[t] = r / sqrt(mean(r^2) + 1e-6), r = x[t] + y[t], an RMS norm
 * with unit weight. No counterpart in the reference, whose MoE layers are joined by its attention
 * blocks. x_next may be x. The operation order is fixed (see frx_chain.cu) so that a CPU
 * restatement gives the same bits. T rows of n floats. */
int frx_chain_rmsnorm_unit(const float* x, const float* y, float* x_next, int T, int n, frx_stream_t stream);

/* ---- ggml-layout entry points: gemv:: (kernels/cuda/ggml_gemv.h:26-65) and gemm::
 * (kernels/cuda/ggml_gemm.h:27-68) for ggml type 42 (Q2_0), as the draft head's MoE calls them
 * (arch/qwen4exp/mtp.cu:631-670). Weights are in ggml's own layout, not the tiled one: rows of
 * 18-byte blocks {fp16 d; 16 code bytes, element j in byte j / 4 at bit 2 * (j % 4)}, row-major
 * [nrows][ncols], expert e at w + e * expert_stride_bytes. Activations are ggml Q8_1 rows: blocks
 * {fp16 d; fp16 sum; 32 int8}, every row padded with zeros to a multiple of 512 values. The
 * arithmetic is ggml's vec_dot_q2_0_q8_1 (third_party/ggml/src/ggml-cuda/vecdotq.cuh:728-771): per
 * 32 values an exact integer sum, scaled d_w * d_a * sum in float, chunks added in float. ncols a
 * multiple of 128; pointers and strides multiples of 4 bytes (16 for the bulk-copy fast path); no
 * zeroed tail is needed after the weights (the reference's kernels want gemv::kWeightTailPad).
 * Any other ggml type returns FRX_ERR_SHAPE. bool arguments of the reference are ints here. */
size_t frx_gemv_q8_1_bytes(int64_t ncols, int n_tok);              /* gemv::q8_1_bytes */
int64_t frx_gemv_row_bytes(uint32_t ggml_type, int64_t ncols);     /* gemv::row_bytes; 0 for other types */
/* gemv::quantize_q8_1: x [n_tok][ncols] -> Q8_1 rows (d = amax / 127, q = roundf(x / d)) */
int frx_gemv_quantize_q8_1(const float* x, int64_t ncols, int n_tok, void* xq, frx_stream_t stream);
/* gemv::swiglu_q8_1: the same of silu(g) * u */
int frx_gemv_swiglu_q8_1(const float* g, const float* u, int64_t ncols, int n_tok, void* xq, frx_stream_t stream);
/* gemv::matvec_q / gemv::matvec: y [n_tok][nrows] = W x, n_tok <= 8; matvec quantizes x into scratch first */
int frx_gemv_matvec_q(uint32_t ggml_type, const void* W, const void* xq, float* y, int64_t ncols, int64_t nrows, int n_tok,
                      frx_stream_t stream);
int frx_gemv_matvec(uint32_t ggml_type, const void* W, const float* x, float* y, int64_t ncols, int64_t nrows, int n_tok, void* scratch,
                    frx_stream_t stream);
/* gemv::moe_q2_0: dst [n_ids][nrows], channel i uses expert ids[i] and activation row 0 (or row i with
 * per_channel_act); with gate, silu(G x) * (W x). */
int frx_gemv_moe_q2_0(const void* w, const void* gate, const void* xq, const int32_t* ids, float* dst, int n_ids, int64_t ncols,
                      int64_t nrows, int64_t slot_stride_bytes, int per_channel_act, frx_stream_t stream);
/* gemv::moe_q: dst [n_tok][k][nrows] = W_{ids[t][j]} x, x = Q8_1 row t (or row t * k + j with
 * act_per_expert); with gate, silu(G x) * (W x). n_tok <= 8. */
int frx_gemv_moe_q(uint32_t ggml_type, const void* w, const void* gate, const void* xq, const int32_t* ids, float* dst, int n_tok, int k,
                   int64_t ncols, int64_t nrows, int64_t expert_stride_bytes, int act_per_expert, frx_stream_t stream);

/* gemm::moe_prepare / moe_run / moe / workspace_bytes: grouped expert products for many tokens.
 * prepare quantizes the activations (row t of x [T][ncols], or row t * K + k of x [T][K][ncols] with
 * x_per_slot) and groups the T * K slots by expert in `ws`, entirely on the device: unlike the
 * reference's it does not wait for the stream. run multiplies one expert tensor: y [T][K][nrows].
 * The plan points into ws, which must stay untouched between prepare and the runs that use it.
 * n_experts <= 4096. ws: 256-byte aligned, frx_gemm_workspace_bytes(ncols, T * K). */
typedef struct frx_gemm_moe_plan {
    uint32_t type;
    int n_experts, K;
    int64_t T, ncols, rows;
    int x_per_slot;
    void* ws;
} frx_gemm_moe_plan;
size_t frx_gemm_workspace_bytes(int64_t ncols, int64_t rows);
int frx_gemm_moe_prepare(frx_gemm_moe_plan* plan, uint32_t ggml_type, int n_experts, const float* x, int x_per_slot, const int32_t* ids,
                         int64_t T, int K, int64_t ncols, void* ws, size_t ws_bytes, frx_stream_t stream);
int frx_gemm_moe_run(const frx_gemm_moe_plan* plan, const void* W, int64_t expert_stride_bytes, float* y, int64_t nrows,
                     frx_stream_t stream);
int frx_gemm_moe(uint32_t ggml_type, const void* W, int64_t expert_stride_bytes, int n_experts, const float* x, int x_per_slot,
                 const int32_t* ids, int64_t T, int K, float* y, int64_t ncols, int64_t nrows, void* ws, size_t ws_bytes,
                 frx_stream_t stream);

/* convert_q8_0_to_q2_0 (arch/qwen4exp/mtp.hpp:40, mtp.cu:129-215) on the device: nblocks64 pairs of
 * Q8_0 blocks {fp16 d; 32 int8} (68 bytes) -> ggml Q2_0 blocks (18 bytes): for each 64 values the
 * scale among 24 candidates (amax / 2.5 .. amax, through fp16) with the least squared error, codes
 * clamp(round(x / d), -1, 2) + 1. Bit-identical to the reference's host function. Device pointers. */
int frx_convert_q8_0_to_q2_0(const void* src_q8_0, void* dst_q2_0, size_t nblocks64, frx_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif
