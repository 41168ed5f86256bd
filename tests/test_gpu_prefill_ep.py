"""Expert-parallel prefill pieces on one GPU: two "ranks" run one after the other over the same
gathered tokens, each with its own expert map (contiguous halves, then a dealt-out placement), on
activations that arrive already quantized; each writes only the slots it holds, the two parts of
every token's weighted sum add up to the oracle's layer output, and the whole pipeline object
(PrefillEp, world size 1) reproduces it too. Needs a GPU."""
import ctypes as C

import numpy as np
import pytest
import torch

from flashrt_b200 import ep, moe, synth
from flashrt_b200.lib import check, lib
from helpers import Experts, cuda, rel_max

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("form,placement", [(1, "ranges"), (2, "ranges"), (1, "dealt")])
def test_two_ranks_in_turn(port, form, placement):
    n, ff, E, K, T = 512, 256, 16, 4, 96
    ex = Experts(port, n, ff, E, shared=False)
    x = synth.activations(T, n, through_bf16=True)
    ids, wts, _ = port.route(synth.zipf_logits(T, E), K)
    ref_out, ref_ys, _ = port.moe_layer(ex.routed_planar(), ex.blob_bytes, None, n, ff, x, ids, wts, None, n_threads=8, want_slots=True)
    xq, xd = moe.quantize_q8(cuda(x))
    assert np.array_equal(xq.cpu().numpy(), port.quantize_q8(x)[0])
    owner = np.arange(E) // (E // 2) if placement == "ranges" else ep.expert_placement(np.bincount(ids.reshape(-1), minlength=E), 2)
    total = torch.zeros(T, n, device="cuda")
    seen = np.zeros(T * K, bool)
    for rank in range(2):
        mine = np.nonzero(owner == rank)[0]
        e_map = np.full(E, -1, np.int32)
        e_map[mine] = np.arange(mine.size)
        # this rank's experts, in ascending id, as its arena would hold them
        local = torch.cat([ex.tiled[e * ex.stride:(e + 1) * ex.stride] for e in mine]).contiguous()
        yd = torch.full((T * K, n), float("nan"), device="cuda")
        ws = moe.workspace(moe.moe_q2.workspace_bytes(T, K, n, ff, mine.size))
        wp, wb = moe._ws_ptr(ws)
        d_map, d_ids, d_wts = cuda(e_map), cuda(ids), cuda(wts)      # kept alive for the calls
        check(lib.frx_moe_prefill_q8_ep(C.c_void_p(local.data_ptr()), ex.stride, mine.size, moe._ptr(d_map), E, n, ff, moe._ptr(xq), moe._ptr(xd),
                                        moe._ptr(d_ids), T, K, moe._ptr(yd), wp, wb, moe._stream(), form))
        part = torch.empty(T, n, device="cuda")
        check(lib.frx_moe_combine_partial(moe._ptr(part), moe._ptr(yd), moe._ptr(d_wts), moe._ptr(d_ids), moe._ptr(d_map), n, K, T, moe._stream()))
        torch.cuda.synchronize()
        moe.workspace_status(ws)
        ys = yd.cpu().numpy()
        held = (e_map[ids.reshape(-1)] >= 0)
        assert np.all(np.isnan(ys[~held])), "a slot held elsewhere was written"
        assert max(rel_max(ys[s], ref_ys[s]) for s in np.nonzero(held)[0]) < 1e-5
        seen |= held
        total += part
    assert seen.all()
    assert rel_max(total.cpu().numpy(), ref_out) < 1e-5


def test_pipeline_object_on_one_rank(port):
    n, ff, E, K, T = 512, 256, 16, 4, 120
    ex = Experts(port, n, ff, E, shared=False)
    x, lg = synth.activations(T, n, through_bf16=True), synth.router_logits(T, E)
    ids, wts, _ = port.route(lg, K)
    pipe = ep.PrefillEp(ex.base, ex.stride, E, n, ff, T, K, chunks=3)
    out, ids_o, _ = pipe.run(cuda(x), cuda(lg))
    torch.cuda.synchronize()
    pipe.status()
    assert np.array_equal(ids_o.cpu().numpy(), ids)
    want = port.moe_layer(ex.routed_planar(), ex.blob_bytes, None, n, ff, x, ids, wts, None, n_threads=8)
    assert rel_max(out.cpu().numpy(), want) < 1e-5
    out2, _, _ = pipe.run(cuda(x), cuda(lg))          # buffers are reused from call to call
    torch.cuda.synchronize()
    assert torch.equal(out2, out)
