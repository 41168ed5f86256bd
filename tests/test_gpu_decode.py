"""The decode-sized MoE layer on the GPU against the CPU oracle (the reference's scalar arithmetic).

Bars: hidden activations and their Q8 codes bit-exact; per-slot expert outputs and the combined
layer output within max|diff| / RMS(ref) <= 1e-3 (the bound asked of the path; what is observed is
around 1e-7, because only the exp() inside SwiGLU can differ in its last bit). Needs a GPU."""
import os

import numpy as np
import pytest
import torch

from flashrt_b200 import moe, synth
from helpers import Experts, cuda, rel_max

pytestmark = pytest.mark.gpu
TOL = 1e-3
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "q2moe_small.npz")


def run_decode(ex, x, ids, wts, gate=None, shared=True, want_ws=False):
    T, K = ids.shape
    ws = moe.workspace(moe.moe_decode_workspace_bytes(T, K, ex.n, ex.ff))
    yslot = torch.full((T * K, ex.n), float("nan"), device="cuda")
    out = moe.moe_decode(ex.base, ex.stride, ex.E, ex.shared_ptr if shared else None, ex.n, ex.ff, cuda(x), cuda(ids), cuda(wts),
                         None if gate is None else cuda(gate), yslot=yslot, ws=ws)
    moe.workspace_status(ws)
    if want_ws:
        return out.cpu().numpy(), yslot.cpu().numpy(), ws
    return out.cpu().numpy(), yslot.cpu().numpy()


def test_fixture_from_reference():
    # per-slot outputs against vectors the reference's scalar expert_ffn produced; layer output
    # against the reference's moe_cpu
    g = np.load(GOLD)
    n, ff, E, K, T = (int(v) for v in g["shape"])
    planar = g["planar"]
    tiled = moe.tile_experts(cuda(planar.reshape(-1)), n, ff, E)
    ws = moe.workspace(moe.moe_decode_workspace_bytes(T, K, n, ff))
    yslot = torch.empty(T * K, n, device="cuda")
    out = moe.moe_decode(tiled.data_ptr(), moe.expert_stride(n, ff), E, None, n, ff, cuda(g["x"]), cuda(g["ids"]), cuda(g["wts"]),
                         None, yslot=yslot, ws=ws)
    moe.workspace_status(ws)
    ys = yslot.cpu().numpy()
    for t in range(4):
        for k in range(K):
            assert rel_max(ys[t * K + k], g["expert_ffn_scalar"][g["ids"][t, k]][t]) < 1e-5
    assert rel_max(out.cpu().numpy(), g["moe_cpu_out"]) < TOL
    xq = moe.decode_workspace_view(ws, T, K, n, ff, "xq").cpu().numpy()
    xd = moe.decode_workspace_view(ws, T, K, n, ff, "xd").cpu().numpy()
    assert np.array_equal(xq, g["xq"]) and np.array_equal(xd, g["xd"])


@pytest.mark.parametrize("T", [1, 3, 4, 16, 64])
def test_layer_config_shape(port, T):
    # the benchmark's layer shape with fewer experts (the CPU oracle has to finish in seconds)
    n, ff, E, K = 2048, 512, 48, 10
    ex = Experts(port, n, ff, E, direct=True)
    x = synth.activations(T, n)
    ids, wts, _ = port.route(synth.router_logits(T, E), K)
    gate = np.random.default_rng(3).standard_normal(T).astype(np.float32)
    from flashrt_b200.lib import check, lib
    out_d, ys_d = run_decode(ex, x, ids, wts, gate)            # the default: down forms and quantizes the hidden rows itself
    try:                                                       # with the separate quantizer the hidden rows pass through the workspace
        check(lib.frx_debug_set_fold_quant(0))
        out, ys, ws = run_decode(ex, x, ids, wts, gate, want_ws=True)
    finally:
        check(lib.frx_debug_set_fold_quant(1))
    assert np.array_equal(ys_d, ys) and np.array_equal(out_d, out)
    try:                                                       # the FFN as one kernel: the hidden rows stay on chip
        check(lib.frx_debug_set_fused_ffn(1))
        out_f, ys_f = run_decode(ex, x, ids, wts, gate)
    finally:
        check(lib.frx_debug_set_fused_ffn(0))
    assert np.array_equal(ys_f, ys) and np.array_equal(out_f, out)
    ref_out, ref_ys, ref_sh = port.moe_layer(ex.routed_planar(), ex.blob_bytes, ex.shared_planar, n, ff, x, ids, wts, gate,
                                             n_threads=8, want_slots=True)
    # hidden activations: Q8 codes bit-exact for a sample of slots
    h = moe.decode_workspace_view(ws, T, K, n, ff, "h").cpu().numpy()
    xq, xd = port.quantize_q8(x)
    hq_gpu = moe.decode_workspace_view(ws, T, K, n, ff, "hq").cpu().numpy()
    hd_gpu = moe.decode_workspace_view(ws, T, K, n, ff, "hd").cpu().numpy()
    assert np.array_equal(moe.decode_workspace_view(ws, T, K, n, ff, "xq").cpu().numpy(), xq)
    assert np.array_equal(moe.decode_workspace_view(ws, T, K, n, ff, "xd").cpu().numpy(), xd)
    for s in list(range(0, T * K, max(1, T * K // 12)))[:12]:
        t = s // K
        _, rh, rhq, rhd = port.expert_ffn(ex.planar[ids[t, s % K]], n, ff, xq[t], xd[t], want_hidden=True)
        assert np.array_equal(hq_gpu[s], rhq) and np.array_equal(hd_gpu[s], rhd)
        assert np.abs(h[s] - rh).max() <= 1e-6 * np.abs(rh).max()
    # the matvec arithmetic is bit-faithful: hidden values differ from the oracle's only where the
    # GPU's exp() and the C library's round differently (a small fraction), and wherever a slot's
    # hidden values are all identical, its output row is identical too
    same_h = h[:T * K].view(np.int32) == np.stack([port.expert_ffn(ex.planar[ids[s // K, s % K]], n, ff, xq[s // K], xd[s // K],
                                                                    want_hidden=True)[1] for s in range(T * K)]).view(np.int32)
    assert same_h.mean() > 0.99, same_h.mean()
    exact_slots = np.nonzero(same_h.all(axis=1))[0]
    assert len(exact_slots) > 0
    for s in exact_slots:
        assert np.array_equal(ys[s], ref_ys[s])
    worst = max(rel_max(ys[s], ref_ys[s]) for s in range(T * K))
    assert worst < TOL, worst
    assert worst < 1e-5, worst            # what bit-faithful arithmetic actually gives
    assert rel_max(out, ref_out) < 1e-5
    ysh = moe.decode_workspace_view(ws, T, K, n, ff, "ysh").cpu().numpy()
    assert rel_max(ysh, ref_sh) < 1e-5


@pytest.mark.parametrize("n,ff,E,K,T", [(256, 128, 8, 3, 5), (2560, 640, 12, 4, 3), (128, 128, 4, 1, 2), (512, 256, 40, 32, 9), (384, 640, 6, 2, 70)])
def test_other_shapes(port, n, ff, E, K, T):
    # includes the reference model's shape (2560 / 640), K = 32, and more tokens than one chunk
    ex = Experts(port, n, ff, E)
    x = synth.activations(T, n)
    ids, wts, _ = port.route(synth.router_logits(T, E), K)
    out, ys = run_decode(ex, x, ids, wts, None)
    ref_out, ref_ys, _ = port.moe_layer(ex.routed_planar(), ex.blob_bytes, ex.shared_planar, n, ff, x, ids, wts, None, n_threads=8,
                                        want_slots=True)
    assert max(rel_max(ys[s], ref_ys[s]) for s in range(T * K)) < 1e-5
    assert rel_max(out, ref_out) < 1e-5


def test_without_shared_expert_and_edge_inputs(port):
    n, ff, E, K, T = 256, 128, 8, 3, 6
    ex = Experts(port, n, ff, E)
    x = synth.activations(T, n)
    x[1] = 0.0                      # an all-zero token: zero scales, zero output
    x[2] *= 1e-4
    x[3] *= 1e3
    ids, wts, _ = port.route(synth.router_logits(T, E), K)
    ids[4] = ids[0]                 # two tokens with identical experts
    out, ys = run_decode(ex, x, ids, wts, None, shared=False)
    ref_out, ref_ys, _ = port.moe_layer(ex.routed_planar(), ex.blob_bytes, None, n, ff, x, ids, wts, None, want_slots=True)
    assert np.all(out[1] == 0) and np.all(ref_out[1] == 0)
    for s in range(T * K):
        if s // K != 1:
            assert rel_max(ys[s], ref_ys[s]) < 1e-5
    assert rel_max(out, ref_out) < 1e-5


def test_window_bit_identical_to_single_token_calls(port):
    # tests/test_moe_hits.cpp:125-165: grouping tokens by expert must not change any value
    n, ff, E, K, T = 2048, 512, 16, 10, 5
    ex = Experts(port, n, ff, E, direct=True)
    x = synth.activations(T, n)
    ids, wts, _ = port.route(synth.router_logits(T, E), K)
    out, ys = run_decode(ex, x, ids, wts, None)
    for t in range(T):
        o1, y1 = run_decode(ex, x[t:t + 1], ids[t:t + 1], wts[t:t + 1], None)
        assert np.array_equal(y1, ys[t * K:(t + 1) * K])
        assert np.array_equal(o1[0], out[t])


def test_bad_expert_id_is_reported(port):
    n, ff, E, K, T = 256, 128, 8, 3, 2
    ex = Experts(port, n, ff, E)
    ids = np.array([[0, 1, 2], [3, 99, 4]], np.int32)
    wts = np.full((T, K), 1 / 3, np.float32)
    ws = moe.workspace(moe.moe_decode_workspace_bytes(T, K, n, ff))
    moe.moe_decode(ex.base, ex.stride, E, None, n, ff, cuda(synth.activations(T, n)), cuda(ids), cuda(wts), None, ws=ws)
    with pytest.raises(moe.FrxError, match="expert id out of range"):
        moe.workspace_status(ws)


def test_layer_with_router_and_host_entry(port):
    n, ff, E, K, T = 512, 256, 32, 4, 7
    ex = Experts(port, n, ff, E)
    x, lg = synth.activations(T, n), synth.router_logits(T, E)
    gate = np.linspace(-2, 2, T).astype(np.float32)
    ids, wts, _ = port.route(lg, K)
    ref_out = port.moe_layer(ex.routed_planar(), ex.blob_bytes, ex.shared_planar, n, ff, x, ids, wts, gate)
    ids_out = torch.empty(T, K, dtype=torch.int32, device="cuda")
    wts_out = torch.empty(T, K, device="cuda")
    out = moe.moe_layer(ex.base, ex.stride, E, ex.shared_ptr, n, ff, cuda(x), cuda(lg), cuda(gate), K, ids_out=ids_out, wts_out=wts_out)
    assert np.array_equal(ids_out.cpu().numpy(), ids)
    assert np.abs(wts_out.cpu().numpy() - wts).max() < 1e-6
    assert rel_max(out.cpu().numpy(), ref_out) < 1e-5
    ws = moe.workspace(moe.moe_layer_host_workspace_bytes(T, K, n, ff, E))
    out_h = torch.empty(T, n).pin_memory()
    moe.moe_layer_host(ex.base, ex.stride, E, ex.shared_ptr, n, ff, torch.from_numpy(x).pin_memory(), torch.from_numpy(lg).pin_memory(),
                       torch.from_numpy(gate).pin_memory(), K, out_h, ws)
    assert np.array_equal(out_h.numpy(), out.cpu().numpy())
    # the pipelined many-layer form: 9 "layers" (more than its four staging slots) over the same
    # experts with different activations, identical to one call per layer
    L = 9
    xs = [torch.from_numpy(synth.activations(T, n, seed=100 + l)).pin_memory() for l in range(L)]
    ls = [torch.from_numpy(synth.router_logits(T, E, seed=200 + l)).pin_memory() for l in range(L)]
    gs = [torch.from_numpy(gate + 0.1 * l).pin_memory() if l % 2 == 0 else None for l in range(L)]
    outs = [torch.empty(T, n).pin_memory() for _ in range(L)]
    wsl = moe.workspace(moe.moe_layers_host_workspace_bytes(T, K, n, ff, E))
    moe.moe_layers_host([ex.base] * L, ex.stride, E, [ex.shared_ptr] * L, n, ff, xs, ls, gs, K, outs, wsl)
    for l in range(L):
        want = torch.empty(T, n).pin_memory()
        moe.moe_layer_host(ex.base, ex.stride, E, ex.shared_ptr, n, ff, xs[l], ls[l], gs[l], K, want, ws)
        assert np.array_equal(outs[l].numpy(), want.numpy()), l
    moe.workspace_status(wsl)


def test_combine_in_hit_order(port):
    # k_moe_combine semantics: k order, hit_n rows, shared expert times sigmoid(gate)
    rng = np.random.default_rng(4)
    T, K, n = 3, 5, 384
    yh = rng.standard_normal((T, K, n), dtype=np.float32)
    w = rng.random((T, K), dtype=np.float32)
    hit_n = np.array([5, 3, 0], np.int32)
    sh = rng.standard_normal((T, n), dtype=np.float32)
    gate = np.array([0.3, -1.2, 4.0], np.float32)
    out = moe.moe_combine(cuda(yh), cuda(w), cuda(hit_n), cuda(sh), cuda(gate)).cpu().numpy()
    for t in range(T):
        acc = np.zeros(n, np.float32)
        for k in range(hit_n[t]):
            acc = acc + w[t, k] * yh[t, k]
        g = np.float32(1.0) / (np.float32(1.0) + np.exp(-gate[t], dtype=np.float32))
        acc = acc + sh[t] * g
        assert np.abs(out[t] - acc).max() <= 1e-6 * max(1.0, np.abs(acc).max())


def test_expert_parallel_partial_sums_add_up(port):
    # two expert ranges computed one after the other on one GPU (what two ranks would compute):
    # the partial sums add up to the full layer, and each range writes only its own slots
    from flashrt_b200 import ep
    n, ff, E, K, T = 512, 256, 16, 4, 9
    ex = Experts(port, n, ff, E)
    x = synth.activations(T, n)
    ids, wts, _ = port.route(synth.router_logits(T, E), K)
    gate = np.linspace(-1, 1, T).astype(np.float32)
    full, ys_full = run_decode(ex, x, ids, wts, gate)
    total = np.zeros((T, n), np.float32)
    for rank in range(2):
        lo, hi = ep.expert_range(rank, 2, E)
        ws = moe.workspace(moe.moe_decode_workspace_bytes(T, K, n, ff))
        out = torch.empty(T, n, device="cuda")
        yslot = torch.full((T * K, n), float("nan"), device="cuda")
        ep.moe_decode_ep(ex.base + lo * ex.stride, ex.stride, E, lo, hi, ex.shared_ptr if rank == 0 else None, n, ff, cuda(x), cuda(ids),
                         cuda(wts), cuda(gate) if rank == 0 else None, out, ws, yslot=yslot)
        moe.workspace_status(ws)
        ys = yslot.cpu().numpy()
        local = ((ids >= lo) & (ids < hi)).reshape(-1)
        assert np.array_equal(ys[local], ys_full[local])
        assert np.all(np.isnan(ys[~local]))
        total += out.cpu().numpy()
    assert rel_max(total, full) < 1e-6


def test_layer_replayed_from_a_cuda_graph_with_new_inputs(port):
    # the decode entry takes every per-step value from device memory, so one captured graph serves
    # every step: replay with new activations and logits in the same buffers, compare with direct calls
    n, ff, E, K, T = 512, 256, 32, 4, 3      # a verify window: 1 token + 2 drafts
    ex = Experts(port, n, ff, E)
    x, lg, gate = torch.empty(T, n, device="cuda"), torch.empty(T, E, device="cuda"), torch.empty(T, device="cuda")
    out = torch.empty(T, n, device="cuda")
    ws = moe.workspace(moe.moe_layer_workspace_bytes(T, K, n, ff))

    def fill(seed):
        x.copy_(cuda(synth.activations(T, n, seed=seed)))
        lg.copy_(cuda(synth.router_logits(T, E, seed=seed + 1)))
        gate.copy_(cuda(np.linspace(-1, 1, T).astype(np.float32) * seed))

    fill(1)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):   # first call outside capture: shared-memory attributes are set once per device
        moe.moe_layer(ex.base, ex.stride, E, ex.shared_ptr, n, ff, x, lg, gate, K, out=out, ws=ws)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        moe.moe_layer(ex.base, ex.stride, E, ex.shared_ptr, n, ff, x, lg, gate, K, out=out, ws=ws)
    for seed in (2, 3, 4):
        fill(seed)
        graph.replay()
        torch.cuda.synchronize()
        got = out.clone()
        want = moe.moe_layer(ex.base, ex.stride, E, ex.shared_ptr, n, ff, x, lg, gate, K)
        assert torch.equal(got, want), seed
    moe.workspace_status(ws)


def test_narrow_and_wide_item_forms_give_the_same_bits(port):
    # items of at most four tokens take another arrangement of the same products (two row groups in
    # one MMA accumulator); with the knob off every item takes the eight-token form
    from flashrt_b200.lib import check, lib
    n, ff, E, K, T = 1024, 256, 96, 6, 40        # 2.5 tokens per expert: narrow and wide items mixed
    ex = Experts(port, n, ff, E, direct=True)
    x = synth.activations(T, n)
    ids, wts, _ = port.route(synth.router_logits(T, E), K)
    gate = np.linspace(-1, 1, T).astype(np.float32)
    try:
        check(lib.frx_debug_set_narrow_items(0))
        out_w, ys_w = run_decode(ex, x, ids, wts, gate)
    finally:
        check(lib.frx_debug_set_narrow_items(1))
    out_n, ys_n = run_decode(ex, x, ids, wts, gate)                # narrow items (the default)
    assert np.array_equal(ys_n, ys_w) and np.array_equal(out_n, out_w)
    for forms, fold in ((0, 1), (1, 1), (3, 1), (2, 0), (3, 0)):   # two or four row groups per task, per kernel (default: 2);
        try:                                                       # hidden rows made by down itself or by the separate quantizer
            check(lib.frx_debug_set_four_group_tasks(forms))
            check(lib.frx_debug_set_fold_quant(fold))
            out_2, ys_2 = run_decode(ex, x, ids, wts, gate)
        finally:
            check(lib.frx_debug_set_four_group_tasks(2))
            check(lib.frx_debug_set_fold_quant(1))
        assert np.array_equal(ys_2, ys_w) and np.array_equal(out_2, out_w), (forms, fold)
    for weight, per_item in ((0, 256), (16, 0), (40, 1024)):       # how down's tasks are shared out among its blocks (default: 22, 256)
        try:
            check(lib.frx_debug_set_down_task_weight(weight))
            check(lib.frx_debug_set_down_item_weight(per_item))
            out_2, ys_2 = run_decode(ex, x, ids, wts, gate)
        finally:
            check(lib.frx_debug_set_down_task_weight(22))
            check(lib.frx_debug_set_down_item_weight(256))
        assert np.array_equal(ys_2, ys_w) and np.array_equal(out_2, out_w), (weight, per_item)
    for bufs in ((0, 0), (2, 2), (4, 3)):                          # the FFN as one kernel, with different numbers of item buffers
        try:
            check(lib.frx_debug_set_fused_ffn(1))
            check(lib.frx_debug_set_ffn_buffers(*bufs))
            out_f, ys_f = run_decode(ex, x, ids, wts, gate)
        finally:
            check(lib.frx_debug_set_ffn_buffers(0, 0))
            check(lib.frx_debug_set_fused_ffn(0))
        assert np.array_equal(ys_f, ys_w) and np.array_equal(out_f, out_w), bufs
    ref_out, ref_ys, _ = port.moe_layer(ex.routed_planar(), ex.blob_bytes, ex.shared_planar, n, ff, x, ids, wts, gate, n_threads=8,
                                        want_slots=True)
    assert max(rel_max(ys_n[s], ref_ys[s]) for s in range(T * K)) < 1e-5
    assert rel_max(out_n, ref_out) < 1e-5


@pytest.mark.parametrize("T", [3, 64])
def test_full_layer_shape_on_a_slot_sample(port, T):
    # BASELINE configs[1] (and the 3-token verify window of configs[3]) at the full shape: 512 experts
    # + shared, hidden 2048, intermediate 512, top-10. The oracle computes a sample of slots (every
    # expert FFN is independent) and the combined output of two tokens.
    n, ff, E, K = 2048, 512, 512, 10
    ex = Experts(port, n, ff, E, direct=True)
    x, lg = synth.activations(T, n), synth.router_logits(T, E)
    gate = np.random.default_rng(5).standard_normal(T).astype(np.float32)
    ids, wts, _ = port.route(lg, K)
    ids_o = torch.empty(T, K, dtype=torch.int32, device="cuda")
    wts_o = torch.empty(T, K, device="cuda")
    ws = moe.workspace(moe.moe_layer_workspace_bytes(T, K, n, ff))
    out = moe.moe_layer(ex.base, ex.stride, E, ex.shared_ptr, n, ff, cuda(x), cuda(lg), cuda(gate), K, ids_out=ids_o, wts_out=wts_o, ws=ws)
    moe.workspace_status(ws)
    assert np.array_equal(ids_o.cpu().numpy(), ids)                    # router ids bit-exact
    _, ys = run_decode(ex, x, ids, wts, gate)
    xq, xd = port.quantize_q8(x)
    rng = np.random.default_rng(6)
    for s in rng.choice(T * K, size=min(24, T * K), replace=False):
        t, k = divmod(int(s), K)
        want = port.expert_ffn(ex.planar[ids[t, k]], n, ff, xq[t], xd[t])
        assert rel_max(ys[s], want) < 1e-5, (s, rel_max(ys[s], want))
    got = out.cpu().numpy()
    for t in (0, T - 1):
        by_id = np.argsort(ids[t])          # the layer sums a token's experts in ascending id
        want = port.moe_layer(np.ascontiguousarray(ex.planar[ids[t][by_id]]), ex.blob_bytes, ex.shared_planar, n, ff, x[t:t + 1],
                              np.arange(K, dtype=np.int32)[None], wts[t:t + 1][:, by_id], gate[t:t + 1])
        assert rel_max(got[t:t + 1], want) < 1e-5


def test_stream_stamps_are_written_and_ordered(port):
    # the measurement aid: four time stamps per block of the two streaming kernels, four of the head
    from flashrt_b200.lib import check, lib
    import ctypes as C
    n, ff, E, K, T = 1024, 256, 96, 6, 40
    ex = Experts(port, n, ff, E, direct=True)
    x = synth.activations(T, n)
    ids, wts, _ = port.route(synth.router_logits(T, E), K)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    st = torch.zeros((2 * sms + 1) * 4, dtype=torch.int64, device="cuda")
    want, _ = run_decode(ex, x, ids, wts, None)
    try:
        check(lib.frx_debug_set_stream_stamps(C.c_void_p(st.data_ptr())))
        got, _ = run_decode(ex, x, ids, wts, None)
    finally:
        check(lib.frx_debug_set_stream_stamps(None))
    assert np.array_equal(got, want)
    s = st.cpu().numpy()
    gu, dn, head = s[:sms * 4].reshape(sms, 4), s[sms * 4:2 * sms * 4].reshape(sms, 4), s[2 * sms * 4:]
    busy = gu[:, 3] > 0                                   # blocks that had tasks
    assert busy.any() and (np.diff(gu[busy], axis=1) >= 0).all()
    busy = dn[:, 3] > 0
    assert busy.any() and (np.diff(dn[busy], axis=1) >= 0).all()
    assert (np.diff(head) >= 0).all() and head[0] > 0
    assert head[3] <= gu[gu[:, 1] > 0, 1].min()           # gate/up's wait returns after the head has written the items
