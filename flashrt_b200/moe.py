"""Host-side mirror of the reference's operator interface for the Q2_0 MoE expert path.

Function names and argument meanings follow the reference (``moe_route_topk``, ``moe_hits``,
``moe_q2.run`` / ``workspace_bytes``, ``ExpertArena.blob``, ``q2_0`` helpers); errors surface as
``FrxError`` where the reference throws ``std::runtime_error``. torch supplies device memory and
streams only: all compute is in libfrx (hand-written sm_100a kernels), and nothing here runs on
the CPU instead when the library or the GPU is missing.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import lib as _l
from .lib import FrxError, check, lib  # noqa: F401

Q2_0_TYPE = 42          # ggml type id (core/formats.hpp:11-18)
BLOCK, BLOCK_BYTES, Q8_BLOCK = 64, 18, 32


def _ptr(t: torch.Tensor | None):
    return None if t is None else C.c_void_p(t.data_ptr())


def _stream(stream=None):
    s = torch.cuda.current_stream() if stream is None else stream
    return C.c_void_p(s.cuda_stream)


def _dev(*ts):
    for t in ts:
        if t is not None and not (t.is_cuda and t.is_contiguous()):
            raise FrxError(_l.ERR_ARG, "tensors must be contiguous CUDA tensors")


# ---- q2_0 storage ------------------------------------------------------------------------------

def mat_bytes(rows: int, cols: int) -> int:
    return int(lib.frx_q2_mat_bytes(rows, cols))


def expert_bytes(n: int, ff: int) -> int:
    return int(lib.frx_q2_expert_bytes(n, ff))


def expert_stride(n: int, ff: int) -> int:
    return int(lib.frx_q2_expert_stride(n, ff))


def repack(ggml_rows: torch.Tensor, rows: int, cols: int, stream=None) -> torch.Tensor:
    """q2_0::repack on the device: ggml blocks (uint8) -> planar matrix (uint8)."""
    _dev(ggml_rows)
    out = torch.empty(mat_bytes(rows, cols), dtype=torch.uint8, device=ggml_rows.device)
    check(lib.frx_q2_repack(_ptr(ggml_rows), rows, cols, _ptr(out), _stream(stream)))
    return out


def tile_experts(planar: torch.Tensor, n: int, ff: int, n_experts: int, src_stride: int | None = None,
                 dst_stride: int | None = None, out: torch.Tensor | None = None, stream=None) -> torch.Tensor:
    """Planar expert blobs -> the tiled layout the kernels read."""
    _dev(planar, out)
    src_stride = expert_bytes(n, ff) if src_stride is None else src_stride
    dst_stride = expert_stride(n, ff) if dst_stride is None else dst_stride
    if out is None:
        out = torch.zeros(n_experts * dst_stride, dtype=torch.uint8, device=planar.device)
    check(lib.frx_q2_tile_experts(_ptr(planar), src_stride, _ptr(out), dst_stride, n_experts, n, ff, _stream(stream)))
    return out


def untile_experts(tiled: torch.Tensor, n: int, ff: int, n_experts: int, src_stride: int | None = None,
                   dst_stride: int | None = None, stream=None) -> torch.Tensor:
    _dev(tiled)
    src_stride = expert_stride(n, ff) if src_stride is None else src_stride
    dst_stride = expert_bytes(n, ff) if dst_stride is None else dst_stride
    out = torch.zeros(n_experts * dst_stride, dtype=torch.uint8, device=tiled.device)
    check(lib.frx_q2_untile_experts(_ptr(tiled), src_stride, _ptr(out), dst_stride, n_experts, n, ff, _stream(stream)))
    return out


def dequant_expert(tiled_blob: torch.Tensor, n: int, ff: int, stream=None):
    """(q - 1) * d of one tiled expert: gate [ff][n], up [ff][n], down [n][ff] fp32."""
    _dev(tiled_blob)
    dev = tiled_blob.device
    g = torch.empty(ff, n, dtype=torch.float32, device=dev)
    u = torch.empty(ff, n, dtype=torch.float32, device=dev)
    d = torch.empty(n, ff, dtype=torch.float32, device=dev)
    check(lib.frx_q2_dequant_expert(_ptr(tiled_blob), n, ff, _ptr(g), _ptr(u), _ptr(d), _stream(stream)))
    return g, u, d


class ExpertArena:
    """HBM-resident expert arena: ``blob(layer, expert)`` as core/expert_arena.hpp, on the device."""

    def __init__(self, n_layer: int, n_expert: int, n: int, ff: int):
        self._h = C.c_void_p()
        check(lib.frx_arena_create(C.byref(self._h), n_layer, n_expert, n, ff))
        self.n_layer, self.n_expert, self.n, self.ff = n_layer, n_expert, n, ff
        self.stride = int(lib.frx_arena_stride(self._h))
        self.blob_bytes = expert_bytes(n, ff)
        self.layer_stride = self.stride * n_expert

    def base(self) -> int:
        return int(lib.frx_arena_base(self._h))

    def blob(self, layer: int, expert: int) -> int:
        p = lib.frx_arena_blob(self._h, layer, expert)
        if not p:
            raise FrxError(_l.ERR_ARG, f"blob({layer}, {expert}) outside the arena")
        return int(p)

    def total_bytes(self) -> int:
        return int(lib.frx_arena_total_bytes(self._h))

    def load_planar(self, layer: int, expert0: int, count: int, planar: torch.Tensor, src_stride: int | None = None,
                    stream=None) -> None:
        """planar: uint8 tensor (host or device) of `count` planar blobs."""
        if not planar.is_contiguous():
            raise FrxError(_l.ERR_ARG, "planar must be contiguous")
        src_stride = self.blob_bytes if src_stride is None else src_stride
        check(lib.frx_arena_load_planar(self._h, layer, expert0, count, _ptr(planar), src_stride, _stream(stream)))

    def read_planar(self, layer: int, expert0: int, count: int, stream=None) -> torch.Tensor:
        """The planar form of `count` blobs of the arena (the inverse of load_planar): uint8 [count][blob_bytes]."""
        out = torch.zeros(count, self.blob_bytes, dtype=torch.uint8, device="cuda")
        check(lib.frx_q2_untile_experts(C.c_void_p(self.blob(layer, expert0)), self.stride, _ptr(out), self.blob_bytes, count, self.n, self.ff,
                                        _stream(stream)))
        return out

    def close(self) -> None:
        if self._h:
            lib.frx_arena_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Gguf:
    """Metadata and tensor directory of one GGUF file (frx_gguf_open); tensor data stays on disk."""

    def __init__(self, path: str):
        self._h = C.c_void_p()
        check(lib.frx_gguf_open(C.byref(self._h), path.encode()))

    def tensor_names(self) -> list[str]:
        return [lib.frx_gguf_tensor_name(self._h, i).decode() for i in range(lib.frx_gguf_tensor_count(self._h))]

    def get_int(self, key: str, fallback: int = 0) -> int:
        return int(lib.frx_gguf_get_int(self._h, key.encode(), fallback))

    def tensor(self, name: str) -> dict:
        typ, nd, dims, off, nbytes = C.c_uint32(), C.c_int(), (C.c_int64 * 4)(), C.c_uint64(), C.c_uint64()
        check(lib.frx_gguf_tensor(self._h, name.encode(), C.byref(typ), C.byref(nd), dims, C.byref(off), C.byref(nbytes)))
        return {"type": typ.value, "dims": list(dims)[:nd.value], "offset": off.value, "bytes": nbytes.value}

    def close(self) -> None:
        if self._h:
            lib.frx_gguf_close(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def arena_load_gguf(arena: "ExpertArena", gguf: Gguf, layer0: int, n_layer: int, n_expert: int, stream=None) -> tuple[int, float]:
    """Fills arena layers [layer0, layer0 + n_layer) with the Q2_0 experts of the file
    (blk.<l>.ffn_{gate,up,down}_exps.weight): read, repacked and tiled on the device. Returns
    (bytes read, seconds)."""
    nbytes, secs = C.c_uint64(), C.c_double()
    check(lib.frx_arena_load_gguf(arena._h, gguf._h, layer0, n_layer, n_expert, arena.n, arena.ff, _stream(stream), C.byref(nbytes),
                                  C.byref(secs)))
    return int(nbytes.value), float(secs.value)


# ---- routing and quantization ------------------------------------------------------------------

def moe_route_topk(logits: torch.Tensor, k: int, counts: torch.Tensor | None = None,
                   tail_counts: torch.Tensor | None = None, tail_from: int = 1 << 30, stream=None):
    """qwen4exp::moe_route_topk: ids int32 [T][k] (descending probability, ties to the lower
    index) and weights float [T][k]."""
    _dev(logits, counts, tail_counts)
    T, E = logits.shape
    ids = torch.empty(T, k, dtype=torch.int32, device=logits.device)
    wts = torch.empty(T, k, dtype=torch.float32, device=logits.device)
    check(lib.frx_route_topk(_stream(stream), _ptr(logits), T, E, k, _ptr(ids), _ptr(wts), _ptr(counts), _ptr(tail_counts),
                             tail_from))
    return ids, wts


def router_logits(w_router: torch.Tensor, w_gate: torch.Tensor | None, x: torch.Tensor, stream=None):
    """The projection in front of the router (frx_router_logits): w_router bf16 [E][n], w_gate bf16 [n]
    or None, x fp32 [T][n] -> (logits fp32 [T][E], gate_logit fp32 [T] or None)."""
    _dev(w_router, w_gate, x)
    if w_router.dtype != torch.bfloat16 or (w_gate is not None and w_gate.dtype != torch.bfloat16) or x.dtype != torch.float32:
        raise FrxError(_l.ERR_ARG, "router_logits: bf16 weights and fp32 activations")
    T, n = x.shape
    E = w_router.shape[0]
    logits = torch.empty(T, E, dtype=torch.float32, device=x.device)
    gate = torch.empty(T, dtype=torch.float32, device=x.device) if w_gate is not None else None
    check(lib.frx_router_logits(_stream(stream), _ptr(w_router), _ptr(w_gate), _ptr(x), T, E, n, _ptr(logits), _ptr(gate)))
    return logits, gate


def quantize_q8(x: torch.Tensor, stream=None):
    """q2_0::quantize_q8 for every row of x [T][n]: codes int8 [T][n], scales float [T][n/32]."""
    _dev(x)
    T, n = x.shape
    q = torch.empty(T, n, dtype=torch.int8, device=x.device)
    d = torch.empty(T, n // Q8_BLOCK, dtype=torch.float32, device=x.device)
    check(lib.frx_quantize_q8(_stream(stream), _ptr(x), T, n, _ptr(q), _ptr(d)))
    return q, d


# ---- the layer ---------------------------------------------------------------------------------

def moe_decode_workspace_bytes(T: int, K: int, n: int, ff: int) -> int:
    return int(lib.frx_moe_decode_workspace_bytes(T, K, n, ff))


def moe_layer_workspace_bytes(T: int, K: int, n: int, ff: int) -> int:
    return int(lib.frx_moe_layer_workspace_bytes(T, K, n, ff))


def workspace(nbytes: int, device="cuda") -> torch.Tensor:
    """A zeroed, 256-byte-aligned device workspace."""
    return torch.zeros(nbytes + 256, dtype=torch.uint8, device=device)


def _ws_ptr(ws: torch.Tensor):
    p = ws.data_ptr()
    a = (p + 255) // 256 * 256
    return C.c_void_p(a), ws.numel() - (a - p)


def workspace_status(ws: torch.Tensor, stream=None) -> None:
    """Raises FrxError if a kernel of a call that used this workspace reported an error."""
    p, _ = _ws_ptr(ws)
    check(lib.frx_workspace_status(p, _stream(stream)))


def moe_decode(experts: int, stride: int, E: int, shared: int | None, n: int, ff: int, x: torch.Tensor, ids: torch.Tensor,
               wts: torch.Tensor, gate_logit: torch.Tensor | None, out: torch.Tensor | None = None,
               yslot: torch.Tensor | None = None, ws: torch.Tensor | None = None, stream=None) -> torch.Tensor:
    """out[t] = sum_k w * expert(x_t) (+ shared(x_t) * sigmoid(gate_logit[t])). `experts` and
    `shared` are device addresses of tiled blobs (ExpertArena.blob)."""
    _dev(x, ids, wts, gate_logit, out, yslot)
    T, K = ids.shape
    if out is None:
        out = torch.empty(T, n, dtype=torch.float32, device=x.device)
    if ws is None:
        ws = workspace(moe_decode_workspace_bytes(T, K, n, ff), x.device)
    wp, wb = _ws_ptr(ws)
    check(lib.frx_moe_decode(C.c_void_p(experts), stride, E, C.c_void_p(shared) if shared else None, n, ff, _ptr(x), _ptr(ids),
                             _ptr(wts), _ptr(gate_logit), T, K, _ptr(out), _ptr(yslot), wp, wb, _stream(stream)))
    return out


def moe_decode_static(experts: int, stride: int, E: int, shared: int | None, n: int, ff: int, x: torch.Tensor, ids: torch.Tensor,
                      wts: torch.Tensor, gate_logit: torch.Tensor | None, out: torch.Tensor, stream=None) -> torch.Tensor:
    """moe_decode for callers that cannot allocate: no workspace argument, the library's built-in
    4 MiB scratch is used (frx_moe_decode_static). Calls on one device must not overlap."""
    _dev(x, ids, wts, gate_logit, out)
    T, K = ids.shape
    check(lib.frx_moe_decode_static(C.c_void_p(experts), stride, E, C.c_void_p(shared) if shared else None, n, ff, _ptr(x), _ptr(ids),
                                    _ptr(wts), _ptr(gate_logit), T, K, _ptr(out), _stream(stream)))
    return out


def moe_layer(experts: int, stride: int, E: int, shared: int | None, n: int, ff: int, x: torch.Tensor, logits: torch.Tensor,
              gate_logit: torch.Tensor | None, K: int, out: torch.Tensor | None = None, ids_out: torch.Tensor | None = None,
              wts_out: torch.Tensor | None = None, ws: torch.Tensor | None = None, stream=None) -> torch.Tensor:
    """Router + experts + combine in one call (device tensors)."""
    _dev(x, logits, gate_logit, out, ids_out, wts_out)
    T = x.shape[0]
    if out is None:
        out = torch.empty(T, n, dtype=torch.float32, device=x.device)
    if ws is None:
        ws = workspace(moe_layer_workspace_bytes(T, K, n, ff), x.device)
    wp, wb = _ws_ptr(ws)
    check(lib.frx_moe_layer(C.c_void_p(experts), stride, E, C.c_void_p(shared) if shared else None, n, ff, _ptr(x), _ptr(logits),
                            _ptr(gate_logit), T, K, _ptr(out), _ptr(ids_out), _ptr(wts_out), wp, wb, _stream(stream)))
    return out


def moe_layer_host_workspace_bytes(T: int, K: int, n: int, ff: int, E: int) -> int:
    return int(lib.frx_moe_layer_host_workspace_bytes(T, K, n, ff, E))


def moe_layer_host(experts: int, stride: int, E: int, shared: int | None, n: int, ff: int, x_host: torch.Tensor,
                   logits_host: torch.Tensor, gate_logit_host: torch.Tensor | None, K: int, out_host: torch.Tensor,
                   ws: torch.Tensor, stream=None) -> torch.Tensor:
    """The same with host tensors (pinned for speed): copies in, runs, copies out, synchronises."""
    for t in (x_host, logits_host, gate_logit_host, out_host):
        if t is not None and (t.is_cuda or not t.is_contiguous()):
            raise FrxError(_l.ERR_ARG, "moe_layer_host takes contiguous host tensors")
    T = x_host.shape[0]
    wp, wb = _ws_ptr(ws)
    check(lib.frx_moe_layer_host(C.c_void_p(experts), stride, E, C.c_void_p(shared) if shared else None, n, ff, _ptr(x_host),
                                 _ptr(logits_host), _ptr(gate_logit_host), T, K, _ptr(out_host), wp, wb, _stream(stream)))
    return out_host


def moe_layers_host_workspace_bytes(T: int, K: int, n: int, ff: int, E: int) -> int:
    return int(lib.frx_moe_layers_host_workspace_bytes(T, K, n, ff, E))


def moe_layers_host(experts: list[int], stride: int, E: int, shared: list[int | None] | None, n: int, ff: int,
                    x_host: list[torch.Tensor], logits_host: list[torch.Tensor], gate_logit_host: list[torch.Tensor | None] | None,
                    K: int, out_host: list[torch.Tensor], ws: torch.Tensor, stream=None) -> list[torch.Tensor]:
    """L independent layer calls from host tensors in one call (frx_moe_layers_host): the copies of
    neighbouring layers overlap a layer's compute when the host tensors are pinned. Entry l of every
    list belongs to layer l; results are identical to L calls of moe_layer_host."""
    L = len(experts)
    for ts in (x_host, logits_host, out_host):
        if len(ts) != L:
            raise FrxError(_l.ERR_ARG, "moe_layers_host: one entry per layer in every list")
        for t in ts:
            if t.is_cuda or not t.is_contiguous() or t.dtype != torch.float32:
                raise FrxError(_l.ERR_ARG, "moe_layers_host takes contiguous float32 host tensors")
    T = x_host[0].shape[0] if L else 1
    arr = C.c_void_p * max(L, 1)
    ex = arr(*[C.c_void_p(e) for e in experts])
    sh = arr(*[C.c_void_p(e) if e else None for e in shared]) if shared is not None else None
    xs = arr(*[C.c_void_p(t.data_ptr()) for t in x_host])
    ls = arr(*[C.c_void_p(t.data_ptr()) for t in logits_host])
    gs = arr(*[C.c_void_p(t.data_ptr()) if t is not None else None for t in gate_logit_host]) if gate_logit_host is not None else None
    os_ = arr(*[C.c_void_p(t.data_ptr()) for t in out_host])
    wp, wb = _ws_ptr(ws)
    check(lib.frx_moe_layers_host(ex, stride, E, sh, n, ff, xs, ls, gs, L, T, K, os_, wp, wb, _stream(stream)))
    return out_host


def _raw_view(ws: torch.Tensor, off: int, dt, shape):
    wp, _ = _ws_ptr(ws)
    start = wp.value - ws.data_ptr() + off
    count = 1
    for s in shape:
        count *= s
    nbytes = count * torch.empty(0, dtype=dt).element_size()
    return ws[start:start + nbytes].view(dt).view(shape)


def _codes_natural(q: torch.Tensor) -> torch.Tensor:
    """Fragment-order int8 codes [rows][k] -> element order (inverse of the quantizer's permutation)."""
    rows, k = q.shape
    w = q.view(rows, k // 64, 4, 2, 2, 4)          # [row][b][t][s][h][byte]
    return w.permute(0, 1, 3, 4, 2, 5).reshape(rows, k)   # element 64b + 32s + 16h + 4t + byte


def decode_workspace_view(ws: torch.Tensor, T: int, K: int, n: int, ff: int, what: str) -> torch.Tensor:
    """One buffer of a moe_decode workspace (tests, debugging). "xq"/"xd" and "hq"/"hd" are given
    in element order with plain block scales, i.e. as q2_0::quantize_q8 would write them."""
    def off(name):
        o = int(lib.frx_moe_decode_workspace_offset(T, K, n, ff, name.encode()))
        if o == 2 ** 64 - 1:
            raise FrxError(_l.ERR_ARG, f"no workspace buffer named {name}")
        return o
    S = T * K + T
    if what in ("xq", "hq"):
        rows, k = (T, n) if what == "xq" else (S, ff)
        return _codes_natural(_raw_view(ws, off(what), torch.int8, (rows, k)))
    if what in ("xd", "hd"):
        rows, k = (T, n) if what == "xd" else (S, ff)
        a = _raw_view(ws, off("xa" if what == "xd" else "ha"), torch.float32, (rows, k // 32)).clone()
        a[:, 1::2] *= 16.0
        return a
    shapes = {"h": (torch.float32, (S, ff)), "y": (torch.float32, (T * K, n)), "ysh": (torch.float32, (T, n)),
              "order": (torch.int32, (T, K)), "status": (torch.int32, (4,))}
    if what not in shapes:
        raise FrxError(_l.ERR_ARG, f"no workspace buffer named {what}")
    dt, shape = shapes[what]
    return _raw_view(ws, off(what), dt, shape)


def moe_hits_scratch_bytes(K: int, n: int, ff: int, T: int = 1) -> int:
    return int(lib.frx_moe_hits_scratch_bytes(K, n, ff, T))


def moe_hits(hit_ptr: torch.Tensor, hit_n: torch.Tensor, K: int, x: torch.Tensor, n: int, ff: int, yh: torch.Tensor,
             scratch: torch.Tensor | None = None, T: int = 1, stream=None) -> torch.Tensor:
    """qwen4exp::moe_hits: hit_ptr int64 [T][K] device addresses of tiled blobs, hit_n int32 [T];
    yh [T][K][n], rows k >= hit_n[t] are left untouched."""
    _dev(hit_ptr, hit_n, x, yh, scratch)
    if scratch is None:
        scratch = workspace(moe_hits_scratch_bytes(K, n, ff, T), x.device)
    sp, sb = _ws_ptr(scratch)
    check(lib.frx_moe_hits(_ptr(hit_ptr), _ptr(hit_n), K, _ptr(x), n, ff, sp, sb, _ptr(yh), _stream(stream), T))
    return yh


def moe_combine(yh: torch.Tensor, w: torch.Tensor, hit_n: torch.Tensor | None, shexp: torch.Tensor | None,
                gate: torch.Tensor | None, out: torch.Tensor | None = None, stream=None) -> torch.Tensor:
    """k_moe_combine: out[t] = sum_{k < hit_n[t]} w[t][k] * yh[t][k] + shexp[t] * sigmoid(gate[t])."""
    _dev(yh, w, hit_n, shexp, gate, out)
    T, K, n = yh.shape
    if out is None:
        out = torch.empty(T, n, dtype=torch.float32, device=yh.device)
    check(lib.frx_moe_combine(_ptr(out), _ptr(yh), _ptr(w), _ptr(hit_n), _ptr(shexp), _ptr(gate), n, K, T, _stream(stream)))
    return out


class moe_q2:
    """moe_q2::workspace_bytes / moe_q2::run (kernels/cuda/moe_q2.h:21-30)."""

    @staticmethod
    def workspace_bytes(T: int, K: int, n: int, ff: int, E: int) -> int:
        return int(lib.frx_moe_prefill_workspace_bytes(T, K, n, ff, E))

    @staticmethod
    def run(experts: int, stride: int, E: int, n: int, ff: int, x: torch.Tensor, ids: torch.Tensor, yd: torch.Tensor | None = None,
            ws: torch.Tensor | None = None, stream=None, form: str = "auto") -> torch.Tensor:
        """yd[t*K + k] = down(silu(gate x_t) * up x_t) of expert ids[t][k], fp32 [T*K][n].
        form: "auto" (by size), "umma" (tcgen05 / tensor memory) or "stream"."""
        _dev(x, ids, yd)
        T, K = ids.shape
        if yd is None:
            yd = torch.empty(T * K, n, dtype=torch.float32, device=x.device)
        if ws is None:
            ws = workspace(moe_q2.workspace_bytes(T, K, n, ff, E), x.device)
        wp, wb = _ws_ptr(ws)
        fn = {"auto": lib.frx_moe_prefill, "umma": lib.frx_moe_prefill_umma, "stream": lib.frx_moe_prefill_stream}[form]
        check(fn(C.c_void_p(experts), stride, E, n, ff, _ptr(x), _ptr(ids), T, K, _ptr(yd), wp, wb, _stream(stream)))
        return yd

    @staticmethod
    def run_ex(experts: int, stride: int, E: int, n: int, ff: int, x: torch.Tensor, ids: torch.Tensor, block64: bool = False,
               yd_bf16: bool = False, ws: torch.Tensor | None = None, stream=None, form: str = "auto") -> torch.Tensor:
        """moe_q2::run with its two options: activation scale blocks of 64, and bf16 output rows."""
        _dev(x, ids)
        T, K = ids.shape
        yd = torch.empty(T * K, n, dtype=torch.bfloat16 if yd_bf16 else torch.float32, device=x.device)
        if ws is None:
            ws = workspace(moe_q2.workspace_bytes(T, K, n, ff, E), x.device)
        wp, wb = _ws_ptr(ws)
        fn = {"auto": lib.frx_moe_prefill_ex, "umma": lib.frx_moe_prefill_umma_ex, "stream": lib.frx_moe_prefill_stream_ex}[form]
        check(fn(C.c_void_p(experts), stride, E, n, ff, _ptr(x), _ptr(ids), T, K, _ptr(yd), wp, wb, _stream(stream), int(block64), int(yd_bf16)))
        return yd


class gemv:
    """The reference's gemv:: functions for ggml-layout Q2_0 weights (kernels/cuda/ggml_gemv.h:26-65)."""

    @staticmethod
    def q8_1_bytes(ncols: int, n_tok: int) -> int:
        return int(lib.frx_gemv_q8_1_bytes(ncols, n_tok))

    @staticmethod
    def row_bytes(ggml_type: int, ncols: int) -> int:
        return int(lib.frx_gemv_row_bytes(ggml_type, ncols))

    @staticmethod
    def quantize_q8_1(x: torch.Tensor, stream=None) -> torch.Tensor:
        _dev(x)
        n_tok, ncols = x.shape
        xq = torch.empty(gemv.q8_1_bytes(ncols, n_tok), dtype=torch.uint8, device=x.device)
        check(lib.frx_gemv_quantize_q8_1(_ptr(x), ncols, n_tok, _ptr(xq), _stream(stream)))
        return xq

    @staticmethod
    def swiglu_q8_1(g: torch.Tensor, u: torch.Tensor, stream=None) -> torch.Tensor:
        _dev(g, u)
        n_tok, ncols = g.shape
        xq = torch.empty(gemv.q8_1_bytes(ncols, n_tok), dtype=torch.uint8, device=g.device)
        check(lib.frx_gemv_swiglu_q8_1(_ptr(g), _ptr(u), ncols, n_tok, _ptr(xq), _stream(stream)))
        return xq

    @staticmethod
    def moe_q(ggml_type: int, w: torch.Tensor, gate: torch.Tensor | None, xq: torch.Tensor, ids: torch.Tensor, ncols: int, nrows: int,
              expert_stride_bytes: int, act_per_expert: bool, stream=None) -> torch.Tensor:
        """dst [n_tok][k][nrows] = W_{ids[t][j]} x (silu(G x) * (W x) with gate)."""
        _dev(w, gate, xq, ids)
        n_tok, k = ids.shape
        dst = torch.empty(n_tok, k, nrows, dtype=torch.float32, device=w.device)
        check(lib.frx_gemv_moe_q(ggml_type, _ptr(w), _ptr(gate), _ptr(xq), _ptr(ids), _ptr(dst), n_tok, k, ncols, nrows, expert_stride_bytes,
                                 int(act_per_expert), _stream(stream)))
        return dst

    @staticmethod
    def moe_q2_0(w: torch.Tensor, gate: torch.Tensor | None, xq: torch.Tensor, ids: torch.Tensor, ncols: int, nrows: int,
                 slot_stride_bytes: int, per_channel_act: bool, stream=None) -> torch.Tensor:
        _dev(w, gate, xq, ids)
        n_ids = ids.numel()
        dst = torch.empty(n_ids, nrows, dtype=torch.float32, device=w.device)
        check(lib.frx_gemv_moe_q2_0(_ptr(w), _ptr(gate), _ptr(xq), _ptr(ids), _ptr(dst), n_ids, ncols, nrows, slot_stride_bytes,
                                    int(per_channel_act), _stream(stream)))
        return dst

    @staticmethod
    def matvec(ggml_type: int, W: torch.Tensor, x: torch.Tensor, nrows: int, stream=None) -> torch.Tensor:
        _dev(W, x)
        n_tok, ncols = x.shape
        y = torch.empty(n_tok, nrows, dtype=torch.float32, device=x.device)
        scratch = torch.empty(gemv.q8_1_bytes(ncols, n_tok), dtype=torch.uint8, device=x.device)
        check(lib.frx_gemv_matvec(ggml_type, _ptr(W), _ptr(x), _ptr(y), ncols, nrows, n_tok, _ptr(scratch), _stream(stream)))
        return y


class _GemmPlan(C.Structure):
    _fields_ = [("type", C.c_uint32), ("n_experts", C.c_int), ("K", C.c_int), ("T", C.c_int64), ("ncols", C.c_int64), ("rows", C.c_int64),
                ("x_per_slot", C.c_int), ("ws", C.c_void_p)]


class gemm:
    """The reference's grouped expert products for ggml-layout Q2_0 weights (kernels/cuda/ggml_gemm.h:50-68)."""

    @staticmethod
    def workspace_bytes(ncols: int, rows: int) -> int:
        return int(lib.frx_gemm_workspace_bytes(ncols, rows))

    @staticmethod
    def moe_prepare(ggml_type: int, n_experts: int, x: torch.Tensor, x_per_slot: bool, ids: torch.Tensor, ncols: int, ws: torch.Tensor,
                    stream=None) -> _GemmPlan:
        _dev(x, ids)
        T, K = ids.shape
        plan = _GemmPlan()
        wp, wb = _ws_ptr(ws)
        check(lib.frx_gemm_moe_prepare(C.byref(plan), ggml_type, n_experts, _ptr(x), int(x_per_slot), _ptr(ids), T, K, ncols, wp, wb,
                                       _stream(stream)))
        return plan

    @staticmethod
    def moe_run(plan: _GemmPlan, W: torch.Tensor, expert_stride_bytes: int, nrows: int, stream=None) -> torch.Tensor:
        _dev(W)
        y = torch.empty(plan.T, plan.K, nrows, dtype=torch.float32, device=W.device)
        check(lib.frx_gemm_moe_run(C.byref(plan), _ptr(W), expert_stride_bytes, _ptr(y), nrows, _stream(stream)))
        return y


def convert_q8_0_to_q2_0(src: torch.Tensor, stream=None) -> torch.Tensor:
    """qwen4exp::convert_q8_0_to_q2_0 on the device: uint8 [n * 68] Q8_0 block pairs -> uint8 [n * 18] Q2_0 blocks."""
    _dev(src)
    n = src.numel() // 68
    dst = torch.empty(n * 18, dtype=torch.uint8, device=src.device)
    check(lib.frx_convert_q8_0_to_q2_0(_ptr(src), _ptr(dst), n, _stream(stream)))
    return dst


def chain_rmsnorm_unit(x: torch.Tensor, y: torch.Tensor, out: torch.Tensor | None = None, stream=None) -> torch.Tensor:
    """The layer join of the chained-stack benchmark: (x + y) / sqrt(mean((x + y)^2) + 1e-6) per row."""
    _dev(x, y, out)
    T, n = x.shape
    if out is None:
        out = torch.empty_like(x)
    check(lib.frx_chain_rmsnorm_unit(_ptr(x), _ptr(y), _ptr(out), T, n, _stream(stream)))
    return out
