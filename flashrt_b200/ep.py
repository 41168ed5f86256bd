"""Expert-parallel MoE layer over the GPUs of one node: one process per GPU, torch.distributed
(NCCL over NVLink) for the exchange. The reference has no multi-GPU code; this is new.

Decode-sized batches: activations and router logits are replicated, every rank routes (the router
is deterministic, so all ranks agree bit for bit), each rank runs the experts it holds and forms
the weighted partial sum of its slots, and one all-reduce of [T][n] fp32 gives the layer output.
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
    check(lib.frx_route_topk(moe._stream(), moe._ptr(logits), T, E, K, moe._ptr(ids_out), moe._ptr(wts_out), None, None, 1 << 30))
    moe_decode_ep(experts_local, stride, E, e_lo, e_hi, shared, n, ff, x, ids_out, wts_out, gate_logit if shared else None, out, ws)
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(out, group=group)
    return out
