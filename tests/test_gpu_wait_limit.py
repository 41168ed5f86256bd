"""A bounded device wait that runs out: the kernel gives up, reports through the workspace status,
and the next call on the same buffers works. One GPU stands in for two ranks: the "peer" is a second
local communication buffer whose flags nobody raises, so the fused all-reduce of rank 0 waits in
vain for the limit (shortened to a few milliseconds) and returns. Nothing faults or hangs.
Needs a GPU."""
import ctypes as C

import numpy as np
import pytest
import torch

from flashrt_b200 import ep, moe, synth
from flashrt_b200.lib import check, lib
from helpers import Experts, cuda

pytestmark = pytest.mark.gpu


class _Raw:
    """A view of raw device memory for torch.as_tensor."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


def test_fused_all_reduce_gives_up_after_the_limit_and_recovers(port):
    n, ff, E, K, T = 512, 256, 16, 4, 6
    ex = Experts(port, n, ff, E)
    x, lg = synth.activations(T, n), synth.router_logits(T, E)
    ids, wts, _ = port.route(lg, K)
    own, peer = C.c_void_p(), C.c_void_p()
    check(lib.frx_ep_buffer_create(C.byref(own), T, n))
    check(lib.frx_ep_buffer_create(C.byref(peer), T, n))
    nbytes = int(lib.frx_ep_buffer_bytes(T, n))
    foff = int(lib.frx_ep_flags_offset(T, n))
    own_t = torch.as_tensor(_Raw(own.value, nbytes), device="cuda")
    peer_t = torch.as_tensor(_Raw(peer.value, nbytes), device="cuda")
    comm = ep._CommStruct(2, 0, T, n, (C.c_void_p * 8)(own.value, peer.value))
    ws = moe.workspace(moe.moe_layer_workspace_bytes(T, K, n, ff))
    out = torch.full((T, n), float("nan"), device="cuda")
    ids_o = torch.empty(T, K, dtype=torch.int32, device="cuda")
    wts_o = torch.empty(T, K, device="cuda")
    dx, dl = cuda(x), cuda(lg)

    def call():
        wp, wb = moe._ws_ptr(ws)
        # rank 0 of 2 holding every expert, so its partial sum is the whole layer
        check(lib.frx_moe_layer_ep_allreduce(C.c_void_p(ex.base), ex.stride, E, 0, E, C.c_void_p(ex.shared_ptr), n, ff, moe._ptr(dx), moe._ptr(dl),
                                             None, T, K, moe._ptr(out), moe._ptr(ids_o), moe._ptr(wts_o), C.byref(comm), wp, wb, moe._stream()))
        torch.cuda.synchronize()

    try:
        check(lib.frx_debug_set_wait_limit_ns(5_000_000))   # 5 ms
        call()                                              # call 1: the peer never answers
        with pytest.raises(moe.FrxError, match="wait"):
            moe.workspace_status(ws)
        moe.workspace_status(ws)                            # reported once, then clean
        # call 2: the peer's flags are raised by hand and its partial sums (slot 2 & 1 = 0) are all ones
        own_t[foff + 4 * 1024:foff + 8 * 1024].view(torch.int32).fill_(2)
        peer_t[:T * n * 4].view(torch.float32).fill_(1.0)
        torch.cuda.synchronize()
        call()
        moe.workspace_status(ws)
    finally:
        check(lib.frx_debug_set_wait_limit_ns(0))
    want = moe.moe_decode(ex.base, ex.stride, E, ex.shared_ptr, n, ff, dx, ids_o, wts_o, None)   # the routing weights of the call itself
    assert np.array_equal(ids_o.cpu().numpy(), ids)
    assert torch.equal(out, want + 1.0)
    del own_t, peer_t
    check(lib.frx_ep_buffer_destroy(peer))
    check(lib.frx_ep_buffer_destroy(own))
