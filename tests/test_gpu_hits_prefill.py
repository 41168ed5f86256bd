"""moe_hits (per-token lists of expert pointers) and the prefill-sized grouped expert product
(moe_q2::run) on the GPU against the CPU oracle. Needs a GPU."""
import numpy as np
import pytest
import torch

from flashrt_b200 import moe, synth
from helpers import Experts, cuda, rel_max

pytestmark = pytest.mark.gpu


def hits_call(ex, x, slot_of, hit_n):
    T, K = slot_of.shape
    ptrs = torch.tensor((ex.base + slot_of.astype(np.int64) * ex.stride).reshape(-1), dtype=torch.int64, device="cuda")
    yh = torch.full((T, K, ex.n), float("nan"), device="cuda")
    scratch = moe.workspace(moe.moe_hits_scratch_bytes(K, ex.n, ex.ff, T))
    moe.moe_hits(ptrs, cuda(hit_n), K, cuda(x), ex.n, ex.ff, yh, scratch=scratch, T=T)
    moe.workspace_status(scratch)
    return yh.cpu().numpy()


def test_hits_single_token_with_pad_entry(port):
    # tests/test_moe_hits.cpp:62-122: 10 entries over 16 slots, the last a pad entry that must not be written
    n, ff, K = 2560, 640, 10
    ex = Experts(port, n, ff, 16, shared=False, seed=7)
    x = synth.activations(1, n)
    slot_of = np.array([[3, 11, 0, 7, 15, 5, 9, 2, 13, 3]])
    yh = hits_call(ex, x, slot_of, np.array([9], np.int32))
    assert np.all(np.isnan(yh[0, 9]))
    xq, xd = port.quantize_q8(x)
    for k in range(9):
        assert rel_max(yh[0, k], port.expert_ffn(ex.planar[slot_of[0, k]], n, ff, xq[0], xd[0])) < 1e-5


def test_hits_window_bit_identical_to_single_token_calls(port):
    # tests/test_moe_hits.cpp:125-165
    n, ff, K, T = 2560, 640, 10, 3
    ex = Experts(port, n, ff, 16, shared=False, seed=7)
    x = synth.activations(T, n)
    slot_of = np.array([[3, 11, 0, 7, 15, 5, 9, 2, 13, 3], [11, 3, 6, 7, 1, 5, 9, 12, 14, 8], [0, 11, 4, 10, 15, 2, 6, 3, 13, 1]])
    hit_n = np.array([9, 10, 7], np.int32)
    yw = hits_call(ex, x, slot_of, hit_n)
    for t in range(T):
        y1 = hits_call(ex, x[t:t + 1], slot_of[t:t + 1], hit_n[t:t + 1])
        assert np.array_equal(yw[t, :hit_n[t]], y1[0, :hit_n[t]])
        assert np.all(np.isnan(yw[t, hit_n[t]:]))


def test_hits_rejects_large_windows():
    with pytest.raises(moe.FrxError, match="unsupported window"):
        moe.moe_hits(torch.zeros(200 * 10, dtype=torch.int64, device="cuda"), torch.zeros(200, dtype=torch.int32, device="cuda"), 10,
                     torch.zeros(200, 256, device="cuda"), 256, 128, torch.zeros(200, 10, 256, device="cuda"), T=200)


@pytest.mark.parametrize("form", ["stream", "umma"])
@pytest.mark.parametrize("T,E,K,zipf", [(96, 16, 4, False), (300, 24, 6, True), (1, 8, 2, False), (1200, 12, 3, True)])
def test_prefill_per_slot_outputs(port, T, E, K, zipf, form):
    # moe_q2::run contract: yd[t*K + k] = expert ids[t][k] applied to x_t
    n, ff = 256, 128
    ex = Experts(port, n, ff, E, shared=False)
    x = synth.activations(T, n, through_bf16=True)
    lg = synth.zipf_logits(T, E) if zipf else synth.router_logits(T, E)
    ids, wts, _ = port.route(lg, K)
    ws = moe.workspace(moe.moe_q2.workspace_bytes(T, K, n, ff, E))
    yd = moe.moe_q2.run(ex.base, ex.stride, E, n, ff, cuda(x), cuda(ids), ws=ws, form=form)
    moe.workspace_status(ws)
    yd = yd.cpu().numpy()
    _, ref_ys, _ = port.moe_layer(ex.routed_planar(), ex.blob_bytes, None, n, ff, x, ids, wts, None, n_threads=8, want_slots=True)
    assert max(rel_max(yd[s], ref_ys[s]) for s in range(T * K)) < 1e-5


def test_prefill_config_shape_sample(port):
    # layer shape of the benchmark's prefill config, fewer experts and tokens; a sample of slots;
    # the tensor-memory form (chosen by size) and the streaming form must agree to the bit
    n, ff, E, K, T = 2048, 512, 32, 10, 256
    ex = Experts(port, n, ff, E, shared=False, direct=True)
    x = synth.activations(T, n, through_bf16=True)
    ids, wts, _ = port.route(synth.zipf_logits(T, E), K)
    yd = moe.moe_q2.run(ex.base, ex.stride, E, n, ff, cuda(x), cuda(ids)).cpu().numpy()
    assert np.array_equal(yd, moe.moe_q2.run(ex.base, ex.stride, E, n, ff, cuda(x), cuda(ids), form="stream").cpu().numpy())
    xq, xd = port.quantize_q8(x)
    for s in range(0, T * K, 97):
        t, k = divmod(s, K)
        assert rel_max(yd[s], port.expert_ffn(ex.planar[ids[t, k]], n, ff, xq[t], xd[t])) < 1e-5
