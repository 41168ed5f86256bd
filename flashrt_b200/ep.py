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


def moe_layer_ep_fused(comm: EpComm, experts_local: int, stride: int, E: int, e_lo: int, e_hi: int, shared: int | None, n: int, ff: int,
                       x: torch.Tensor, logits: torch.Tensor, gate_logit: torch.Tensor | None, K: int, out: torch.Tensor,
                       ids_out: torch.Tensor, wts_out: torch.Tensor, ws: torch.Tensor, stream=None) -> torch.Tensor:
    """Router on every rank, local experts, and the all-reduce inside the layer's last kernel (peer
    loads over NVLink, partial sums added in rank order on every rank). `out` is the complete layer
    output on every rank. Every rank must make the same sequence of calls."""
    T = x.shape[0]
    wp, wb = moe._ws_ptr(ws)
    check(lib.frx_moe_layer_ep_allreduce(C.c_void_p(experts_local), stride, E, e_lo, e_hi, C.c_void_p(shared) if shared else None, n, ff,
                                         moe._ptr(x), moe._ptr(logits), moe._ptr(gate_logit) if shared else None, T, K, moe._ptr(out),
                                         moe._ptr(ids_out), moe._ptr(wts_out), C.byref(comm.struct), wp, wb, moe._stream(stream)))
    return out


def moe_prefill_ep(experts_local: int, stride: int, E: int, n: int, ff: int, x: torch.Tensor, logits: torch.Tensor, K: int,
                   group=None) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Prefill-sized expert-parallel layer. Tokens are sharded over the ranks (x, logits are this
    rank's tokens), experts too (this rank holds expert_range(rank, world, E), E divisible by the
    world size). Each rank routes its tokens, sends every (token, expert) slot's activations to the
    rank that holds the expert (all-to-all), runs the grouped expert product on what it received,
    returns the results (all-to-all) and sums them with the routing weights.

    Returns (out [T_local][n], ids, wts). One host synchronisation (the split sizes), as the
    reference's grouped path has one."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    if E % world:
        raise moe.FrxError(1, f"moe_prefill_ep: {E} experts do not divide over {world} ranks")
    per = E // world
    T = x.shape[0]
    ids, wts = moe.moe_route_topk(logits, K)
    flat = ids.reshape(-1).to(torch.int64)
    dest = flat // per
    order = torch.sort(dest, stable=True).indices                 # slots grouped by destination rank
    send_counts = torch.bincount(dest, minlength=world)
    recv_counts = torch.empty_like(send_counts)
    if world > 1:
        dist.all_to_all_single(recv_counts, send_counts, group=group)
    else:
        recv_counts.copy_(send_counts)
    sc, rc = send_counts.tolist(), recv_counts.tolist()           # the one host synchronisation
    tok = (order // K)
    send_x = x.index_select(0, tok).contiguous()                  # [S][n]
    send_e = (flat.index_select(0, order) - dest.index_select(0, order) * per).to(torch.int32).contiguous()
    R = int(sum(rc))
    recv_x = torch.empty(R, n, dtype=x.dtype, device=x.device)
    recv_e = torch.empty(R, dtype=torch.int32, device=x.device)
    if world > 1:
        dist.all_to_all_single(recv_x, send_x, output_split_sizes=rc, input_split_sizes=sc, group=group)
        dist.all_to_all_single(recv_e, send_e, output_split_sizes=rc, input_split_sizes=sc, group=group)
    else:
        recv_x, recv_e = send_x, send_e
    y = torch.empty(R, n, dtype=torch.float32, device=x.device)
    if R:
        moe.moe_q2.run(experts_local, stride, per, n, ff, recv_x, recv_e.view(R, 1), yd=y)
    back = torch.empty(T * K, n, dtype=torch.float32, device=x.device)
    if world > 1:
        dist.all_to_all_single(back, y, output_split_sizes=sc, input_split_sizes=rc, group=group)
    else:
        back = y
    yd = torch.empty_like(back)
    yd.index_copy_(0, order, back)                                # slot order t * K + k again
    out = moe.moe_combine(yd.view(T, K, n), wts, None, None, None)
    return out, ids, wts
