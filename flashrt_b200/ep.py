"""Expert-parallel MoE layer over the GPUs of one node: one process per GPU, torch.distributed
(NCCL over NVLink) for the exchange. The reference has no multi-GPU code; this is new.

Decode-sized batches: activations and router logits are replicated, every rank routes (the router
is deterministic, so all ranks agree bit for bit), each rank runs the experts it holds and forms
the weighted partial sum of its slots, and one all-reduce of [T][n] fp32 gives the layer output.
The all-reduce is either NCCL's (moe_layer_ep) or fused into the layer's last kernel over peer
memory (EpComm + moe_layer_ep_fused: no NCCL call on the data path, so steps can be captured in a
CUDA graph).
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from . import moe
from .lib import check, lib


def expert_range(rank: int, world: int, E: int) -> tuple[int, int]:
    """The contiguous block of experts rank holds."""
    return rank * E // world, (rank + 1) * E // world


def moe_decode_ep(experts_local: int, stride: int, E: int, e_lo: int, e_hi: int, shared: int | None, n: int, ff: int,
                  x: torch.Tensor, ids: torch.Tensor, wts: torch.Tensor, gate_logit: torch.Tensor | None, out: torch.Tensor,
                  ws: torch.Tensor, yslot: torch.Tensor | None = None, stream=None) -> torch.Tensor:
    """This rank's partial sum (frx_moe_decode_ep); no communication."""
    T, K = ids.shape
    wp, wb = moe._ws_ptr(ws)
    check(lib.frx_moe_decode_ep(C.c_void_p(experts_local), stride, E, e_lo, e_hi, C.c_void_p(shared) if shared else None, n, ff,
                                moe._ptr(x), moe._ptr(ids), moe._ptr(wts), moe._ptr(gate_logit), T, K, moe._ptr(out), moe._ptr(yslot),
                                wp, wb, moe._stream(stream)))
    return out


def moe_layer_ep(experts_local: int, stride: int, E: int, e_lo: int, e_hi: int, shared: int | None, n: int, ff: int,
                 x: torch.Tensor, logits: torch.Tensor, gate_logit: torch.Tensor | None, K: int, out: torch.Tensor,
                 ids_out: torch.Tensor, wts_out: torch.Tensor, ws: torch.Tensor, group=None) -> torch.Tensor:
    """Router on every rank, local experts, all-reduce of the partial sums. `shared` is the shared
    expert's blob on the one rank that computes it and None elsewhere."""
    T = x.shape[0]
    wp, wb = moe._ws_ptr(ws)
    check(lib.frx_moe_layer_ep(C.c_void_p(experts_local), stride, E, e_lo, e_hi, C.c_void_p(shared) if shared else None, n, ff, moe._ptr(x),
                               moe._ptr(logits), moe._ptr(gate_logit) if shared else None, T, K, moe._ptr(out), moe._ptr(ids_out),
                               moe._ptr(wts_out), wp, wb, moe._stream()))
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(out, group=group)
    return out


class _CommStruct(C.Structure):
    _fields_ = [("world", C.c_int), ("rank", C.c_int), ("max_T", C.c_int), ("n", C.c_int), ("buffer", C.c_void_p * 8)]


class EpComm:
    """The peer-memory communication state of frx_moe_layer_ep_allreduce: one device buffer per
    rank (two slots of partial sums [max_T][n], flag words, counters), every rank's buffer mapped
    into every other rank's address space through CUDA IPC. Collective: every rank of `group`
    constructs it at the same time. The handles travel through torch.distributed (set-up only)."""

    def __init__(self, max_T: int, n: int, group=None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if self.world > 8:
            raise moe.FrxError(1, "EpComm: at most 8 ranks")
        self.max_T, self.n = max_T, n
        self._own = C.c_void_p()
        check(lib.frx_ep_buffer_create(C.byref(self._own), max_T, n))
        handle = C.create_string_buffer(64)
        check(lib.frx_ipc_export(self._own, handle))
        handles = [None] * self.world
        dist.all_gather_object(handles, bytes(handle.raw), group=group)
        self._mapped = []
        ptrs = []
        for q in range(self.world):
            if q == self.rank:
                ptrs.append(self._own.value)
                continue
            m = C.c_void_p()
            check(lib.frx_ipc_open(C.create_string_buffer(handles[q], 64), C.byref(m)))
            self._mapped.append(m)
            ptrs.append(m.value)
        self.struct = _CommStruct(self.world, self.rank, max_T, n, (C.c_void_p * 8)(*ptrs))
        dist.barrier(group=group)   # every rank has mapped every buffer before anyone uses them

    def close(self) -> None:
        """Collective tear-down: every rank of the group calls it at the same point. A rank's buffer
        is freed only after every rank has drained its device (a peer's last kernel may still be
        reading this rank's partial sums over NVLink when this rank's own last kernel has ended)
        and every peer has closed its mapping."""
        if not self._own:
            return
        torch.cuda.synchronize()
        dist.barrier(group=self.group)
        self.close_mappings()
        dist.barrier(group=self.group)
        self.destroy()

    def close_mappings(self) -> None:
        """Step 1 of the tear-down (after every rank has drained its device): unmap the peers' buffers."""
        for m in self._mapped:
            lib.frx_ipc_close(m)
        self._mapped = []

    def destroy(self) -> None:
        """Step 2 (after every rank has unmapped): free this rank's buffer."""
        if self._own:
            lib.frx_ep_buffer_destroy(self._own)
            self._own = C.c_void_p()

    def stamps(self) -> list[int]:
        """SM cycle stamps of this rank's last fused call (frx_ep_debug_stamps)."""
        out = (C.c_longlong * 4)()
        check(lib.frx_ep_debug_stamps(self._own, self.max_T, self.n, out))
        return list(out)


def shared_token_range(rank: int, world: int, T: int, step: int = 4) -> tuple[int, int]:
    """The tokens whose shared-expert rows rank `rank` computes when the shared expert's work is
    dealt among the ranks: contiguous ranges of whole work items (`step` tokens) that partition [0, T)."""
    items = (T + step - 1) // step
    lo, hi = items * rank // world, items * (rank + 1) // world
    return min(lo * step, T), min(hi * step, T)


def moe_layer_ep_fused(comm: EpComm, experts_local: int, stride: int, E: int, e_lo: int, e_hi: int, shared: int | None, n: int, ff: int,
                       x: torch.Tensor, logits: torch.Tensor, gate_logit: torch.Tensor | None, K: int, out: torch.Tensor,
                       ids_out: torch.Tensor, wts_out: torch.Tensor, ws: torch.Tensor, stream=None,
                       shared_tokens: tuple[int, int] | None = None) -> torch.Tensor:
    """Router on every rank, local experts, and the all-reduce inside the layer's last kernel (peer
    loads over NVLink, partial sums added in rank order on every rank). `out` is the complete layer
    output on every rank. Every rank must make the same sequence of calls.
    `shared`: the shared expert's blob on the one rank that applies it to all tokens, or, with
    `shared_tokens` = (t0, t1), on every rank, each applying it to its own tokens (shared_token_range)."""
    T = x.shape[0]
    wp, wb = moe._ws_ptr(ws)
    t0, t1 = shared_tokens if shared_tokens is not None else (0, T)
    check(lib.frx_moe_layer_ep_allreduce_dealt(C.c_void_p(experts_local), stride, E, e_lo, e_hi, C.c_void_p(shared) if shared else None, t0, t1,
                                               n, ff, moe._ptr(x), moe._ptr(logits), moe._ptr(gate_logit) if shared else None, T, K,
                                               moe._ptr(out), moe._ptr(ids_out), moe._ptr(wts_out), C.byref(comm.struct), wp, wb,
                                               moe._stream(stream)))
    return out


def expert_placement(counts, world: int) -> "np.ndarray":
    """Owner rank of every expert, dealing the experts round-robin in order of popularity (counts:
    tokens routed to each expert on some sample), so that the hot experts of a skewed router do not
    all land on one rank. Ties keep the lower expert id first."""
    import numpy as np
    counts = np.asarray(counts)
    order = np.lexsort((np.arange(counts.size), -counts))
    owner = np.empty(counts.size, np.int32)
    owner[order] = np.arange(counts.size, dtype=np.int32) % world
    return owner


class PrefillEp:
    """Expert-parallel prefill of one MoE layer: tokens and experts are both sharded over the ranks.

    Every rank routes and quantizes its own tokens (int8 codes + one float scale per 32 values:
    2,304 bytes per token instead of 8,192), the ranks all-gather the quantized tokens and the
    routing, each rank runs the grouped expert products over all gathered tokens but only over the
    slots whose expert it holds (frx_moe_prefill_q8_ep consumes the quantized form directly), forms
    its part of every token's weighted sum, and a reduce-scatter of those rows gives every rank the
    outputs of its own tokens. The tokens are cut into chunks, and the exchanges run on a second
    stream, so a chunk's all-gather and the previous chunk's reduce-scatter overlap the expert
    products of the chunk in between. Nothing waits for the host: counts stay on the device.

    `owner` [E] gives the rank of every expert (default: contiguous ranges); this rank's experts lie
    at experts_local + i * stride in ascending expert id. All ranks construct it with the same
    arguments and call run() together."""

    def __init__(self, experts_local: int, stride: int, E: int, n: int, ff: int, T_local: int, K: int, owner=None, chunks: int = 4,
                 group=None, device=None, form: int = 0):
        import numpy as np
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        dev = device or torch.device("cuda", torch.cuda.current_device())
        if owner is None:
            owner = np.empty(E, np.int32)
            for r in range(self.world):
                lo, hi = expert_range(r, self.world, E)
                owner[lo:hi] = r
        owner = np.asarray(owner, np.int32)
        mine = np.nonzero(owner == self.rank)[0]
        e_map = np.full(E, -1, np.int32)
        e_map[mine] = np.arange(mine.size, dtype=np.int32)
        self.e_map = torch.from_numpy(e_map).to(dev)
        self.E_local = int(mine.size)
        while chunks > 1 and T_local % chunks:
            chunks -= 1
        self.chunks, self.Tc = chunks, T_local // chunks
        self.experts_local, self.stride, self.E, self.n, self.ff, self.T_local, self.K, self.form = experts_local, stride, E, n, ff, T_local, K, form
        Tg = self.world * self.Tc
        self.meta_w = n // 32 + 2 * K                     # per token: block scales, expert ids, routing weights (32-bit words)
        self.xq_l = torch.empty(chunks, self.Tc, n, dtype=torch.int8, device=dev)
        self.meta_l = torch.empty(chunks, self.Tc, self.meta_w, dtype=torch.int32, device=dev)
        self.xq_g = torch.empty(chunks, Tg, n, dtype=torch.int8, device=dev)
        self.meta_g = torch.empty(chunks, Tg, self.meta_w, dtype=torch.int32, device=dev)
        self.yd = torch.empty(Tg * K, n, dtype=torch.float32, device=dev)
        self.part = torch.empty(2, Tg, n, dtype=torch.float32, device=dev)
        self.out = torch.empty(T_local, n, dtype=torch.float32, device=dev)
        self.ws = moe.workspace(moe.moe_q2.workspace_bytes(Tg, K, n, ff, max(1, self.E_local)), dev)
        self.comm = torch.cuda.Stream(device=dev)
        self.ev_gathered = [torch.cuda.Event() for _ in range(chunks)]
        self.ev_part = [torch.cuda.Event() for _ in range(chunks)]
        self.ev_scattered = [torch.cuda.Event() for _ in range(chunks)]

    def run(self, x: torch.Tensor, logits: torch.Tensor):
        """x [T_local][n], logits [T_local][E] -> (out [T_local][n], ids, wts). out is reused by the next call."""
        n, K, Tc, world = self.n, self.K, self.Tc, self.world
        main = torch.cuda.current_stream()
        ids, wts = moe.moe_route_topk(logits, K)
        for c in range(self.chunks):
            sl = slice(c * Tc, (c + 1) * Tc)
            xd = torch.empty(Tc, n // 32, dtype=torch.float32, device=x.device)
            check(lib.frx_quantize_q8(moe._stream(), moe._ptr(x[sl]), Tc, n, moe._ptr(self.xq_l[c]), moe._ptr(xd)))
            m = self.meta_l[c]
            m[:, :n // 32] = xd.view(torch.int32)
            m[:, n // 32:n // 32 + K] = ids[sl]
            m[:, n // 32 + K:] = wts[sl].view(torch.int32)
            if world > 1:
                self.comm.wait_stream(main)
                with torch.cuda.stream(self.comm):
                    dist.all_gather_into_tensor(self.xq_g[c].view(-1), self.xq_l[c].view(-1), group=self.group)
                    dist.all_gather_into_tensor(self.meta_g[c].view(-1), self.meta_l[c].view(-1), group=self.group)
                    self.ev_gathered[c].record(self.comm)
            else:
                self.xq_g[c].copy_(self.xq_l[c])
                self.meta_g[c].copy_(self.meta_l[c])
        Tg = world * Tc
        wp, wb = moe._ws_ptr(self.ws)
        for c in range(self.chunks):
            if world > 1:
                main.wait_event(self.ev_gathered[c])
            mg = self.meta_g[c]
            xd_g = mg[:, :n // 32].contiguous().view(torch.float32)
            ids_g = mg[:, n // 32:n // 32 + K].contiguous()
            wts_g = mg[:, n // 32 + K:].contiguous().view(torch.float32)
            check(lib.frx_moe_prefill_q8_ep(C.c_void_p(self.experts_local), self.stride, self.E_local, moe._ptr(self.e_map), self.E, n, self.ff,
                                            moe._ptr(self.xq_g[c]), moe._ptr(xd_g), moe._ptr(ids_g), Tg, K, moe._ptr(self.yd), wp, wb,
                                            moe._stream(), self.form))
            part = self.part[c % 2]
            if c >= 2 and world > 1:
                main.wait_event(self.ev_scattered[c - 2])     # the exchange that read this buffer has finished
            check(lib.frx_moe_combine_partial(moe._ptr(part), moe._ptr(self.yd), moe._ptr(wts_g), moe._ptr(ids_g), moe._ptr(self.e_map), n, K,
                                              Tg, moe._stream()))
            dst = self.out[c * Tc:(c + 1) * Tc]
            if world > 1:
                self.ev_part[c].record(main)
                with torch.cuda.stream(self.comm):
                    self.comm.wait_event(self.ev_part[c])
                    dist.reduce_scatter_tensor(dst.view(-1), part.view(-1), group=self.group)
                    self.ev_scattered[c].record(self.comm)
            else:
                dst.copy_(part)
        if world > 1:
            main.wait_stream(self.comm)
        return self.out, ids, wts

    def status(self) -> None:
        moe.workspace_status(self.ws)
