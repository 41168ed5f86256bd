"""The ggml-layout entry points (gemv::quantize_q8_1 / moe_q / moe_q2_0 / matvec, gemm::moe_prepare /
moe_run, convert_q8_0_to_q2_0) on the GPU against the CPU oracle. The shapes follow the reference's
own test of this path (tests/test_moe_q.cpp:53-122: 3 tokens x 4 experts of 8 with a repeated id,
the gate + up pass with fused SwiGLU on one activation per token, the down pass on one activation
per token and expert), with Q2_0 experts. Bars: Q8_1 codes and scales bit-exact; products within
the reference test's 1e-4 relative error (what is observed is ~1e-6: only the order of the float
additions differs); the requantizer bit-exact. Needs a GPU."""
import numpy as np
import pytest
import torch

from flashrt_b200 import moe, synth
from helpers import cuda
from test_ggml_oracle import q8_0_edge_blocks

pytestmark = pytest.mark.gpu
Q2_0 = 42


def rel_l2(a, b):
    a, b = a.astype(np.float64), b.astype(np.float64)
    return float(np.sqrt(((a - b) ** 2).sum() / max((b ** 2).sum(), 1e-30)))


def expert_tensors(rng, E, n, ff):
    gate = np.stack([synth.ggml_blocks(rng, ff, n) for _ in range(E)])   # [E][ff * n/64][18]
    up = np.stack([synth.ggml_blocks(rng, ff, n) for _ in range(E)])
    down = np.stack([synth.ggml_blocks(rng, n, ff) for _ in range(E)])
    return gate.reshape(E, -1), up.reshape(E, -1), down.reshape(E, -1)


def test_quantize_q8_1_bit_exact(port):
    rng = np.random.default_rng(2)
    x = rng.standard_normal((5, 640)).astype(np.float32)
    x[1, 32:64] = 0.0
    x[2] *= 1e-6
    x[3, 7] = 300.0
    # exact halves after scaling: amax 127 makes d = 1, so these land on .5 exactly
    x[4, :32] = np.array([127.0, 0.5, -0.5, 1.5, -2.5] + [0.25] * 27, np.float32)
    got = moe.gemv.quantize_q8_1(cuda(x)).cpu().numpy().reshape(5, -1, 36)
    want = port.quantize_q8_1(x).reshape(5, -1, 36)
    assert got.shape == want.shape
    assert np.array_equal(got[:, :, 0:2], want[:, :, 0:2])        # d
    assert np.array_equal(got[:, :, 4:], want[:, :, 4:])          # codes, the zero padding included
    s_got = got[:, :, 2:4].copy().view(np.float16).astype(np.float32)
    s_want = want[:, :, 2:4].copy().view(np.float16).astype(np.float32)
    assert np.abs(s_got - s_want).max() <= 2e-3 * max(1.0, np.abs(s_want).max())   # the block sum: added in another order


@pytest.mark.parametrize("n,ff", [(2560, 640), (2048, 512), (384, 128)])
def test_moe_q_gate_up_and_down(port, n, ff):
    E, K, T = 8, 4, 3
    rng = np.random.default_rng(11)
    gate, up, down = expert_tensors(rng, E, n, ff)
    ids = np.array([[3, 0, 7, 5], [1, 1, 6, 2], [4, 3, 0, 7]], np.int32)        # a repeated id on purpose
    x = rng.standard_normal((T, n)).astype(np.float32)
    gu_stride, d_stride = gate.shape[1], down.shape[1]
    assert gu_stride == moe.gemv.row_bytes(Q2_0, n) * ff
    dg, du, dd = cuda(gate.reshape(-1)), cuda(up.reshape(-1)), cuda(down.reshape(-1))
    xq = moe.gemv.quantize_q8_1(cuda(x))
    hid = moe.gemv.moe_q(Q2_0, du, dg, xq, cuda(ids), n, ff, gu_stride, False)
    hq = moe.gemv.quantize_q8_1(hid.view(T * K, ff))
    y = moe.gemv.moe_q(Q2_0, dd, None, hq, cuda(ids), ff, n, d_stride, True)
    torch.cuda.synchronize()
    xq_o = port.quantize_q8_1(x)
    assert np.array_equal(xq.cpu().numpy().reshape(xq_o.shape)[:, 4::36], xq_o[:, 4::36])
    hid_o = port.moe_q2_0(up.reshape(-1), gate.reshape(-1), xq_o.reshape(-1), ids, n, ff, gu_stride, False)
    assert rel_l2(hid.cpu().numpy(), hid_o) < 1e-4
    assert rel_l2(hid.cpu().numpy(), hid_o) < 1e-5          # what the same products in another order give
    # the down pass from the GPU's own hidden rows, so it is checked on its own (as the reference's test does)
    hq_o = port.quantize_q8_1(hid.cpu().numpy().reshape(T * K, ff))
    y_o = port.moe_q2_0(down.reshape(-1), None, hq_o.reshape(-1), ids, ff, n, d_stride, True)
    assert rel_l2(y.cpu().numpy(), y_o) < 1e-5
    # moe_q2_0 (one list of channels) and matvec agree with moe_q on the same work
    ch = moe.gemv.moe_q2_0(dd, None, hq, cuda(ids.reshape(-1)), ff, n, d_stride, True)
    assert torch.equal(ch.view(T, K, n), y)
    e = int(ids[2, 1])
    mv = moe.gemv.matvec(Q2_0, dd[e * d_stride:(e + 1) * d_stride], hid.view(T * K, ff)[2 * K + 1:2 * K + 2].contiguous(), n)
    assert torch.equal(mv[0], y[2, 1])


def test_swiglu_q8_1(port):
    rng = np.random.default_rng(5)
    g, u = rng.standard_normal((4, 512)).astype(np.float32) * 3, rng.standard_normal((4, 512)).astype(np.float32)
    got = moe.gemv.swiglu_q8_1(cuda(g), cuda(u)).cpu().numpy().reshape(4, -1, 36)
    h = (g / (1.0 + np.exp(-g)) * u).astype(np.float32)
    want = port.quantize_q8_1(h).reshape(4, -1, 36)
    d_got = got[:, :, 0:2].copy().view(np.float16).astype(np.float32)[:, :, 0]
    d_want = want[:, :, 0:2].copy().view(np.float16).astype(np.float32)[:, :, 0]
    assert np.abs(d_got - d_want).max() <= 2e-3 * d_want.max()          # the fast exponential moves the scale by an fp16 ulp at most
    dq = got[:, :, 4:].view(np.int8).astype(np.int32) - want[:, :, 4:].view(np.int8).astype(np.int32)
    assert np.abs(dq).max() <= 1 and (dq != 0).mean() < 0.02


@pytest.mark.parametrize("per_slot", [False, True])
def test_grouped_products_for_many_tokens(port, per_slot):
    # gemm::moe_prepare + moe_run: 300 tokens x 4 of 12 experts (experts with many, few and no tokens)
    E, K, T, ncols, nrows = 12, 4, 300, 512, 384
    rng = np.random.default_rng(8)
    w = np.stack([synth.ggml_blocks(rng, nrows, ncols) for _ in range(E)]).reshape(E, -1)
    lg = synth.zipf_logits(T, E)
    lg[:, 5] = -50.0                                   # nobody routes to expert 5
    ids = np.argsort(-lg, axis=1)[:, :K].astype(np.int32)
    x = rng.standard_normal((T * K if per_slot else T, ncols)).astype(np.float32)
    ws = moe.workspace(moe.gemm.workspace_bytes(ncols, T * K))
    plan = moe.gemm.moe_prepare(Q2_0, E, cuda(x), per_slot, cuda(ids), ncols, ws)
    y = moe.gemm.moe_run(plan, cuda(w.reshape(-1)), w.shape[1], nrows)
    y2 = moe.gemm.moe_run(plan, cuda(w.reshape(-1)), w.shape[1], nrows)      # a plan serves several tensors
    torch.cuda.synchronize()
    assert torch.equal(y, y2)
    xq = port.quantize_q8_1(x)
    want = np.empty((T, K, nrows), np.float32)
    for t0 in range(0, T, 8):                           # the oracle's moe_q takes the rows in slices
        sl = slice(t0, min(T, t0 + 8))
        rows = xq.reshape(T, K, -1)[sl].reshape(-1) if per_slot else xq[sl].reshape(-1)
        want[sl] = port.moe_q2_0(w.reshape(-1), None, rows, ids[sl], ncols, nrows, w.shape[1], per_slot)
    assert rel_l2(y.cpu().numpy(), want) < 1e-5
    # the grouped form and the small-batch form compute the same products
    t = 17
    xq_t = moe.gemv.quantize_q8_1(cuda(x.reshape(T, K, ncols)[t] if per_slot else x[t:t + 1]))
    mv = moe.gemv.moe_q(Q2_0, cuda(w.reshape(-1)), None, xq_t, cuda(ids[t:t + 1]), ncols, nrows, w.shape[1], per_slot)
    assert rel_l2(mv.cpu().numpy()[0], y.cpu().numpy()[t]) < 1e-6


def test_requantizer_bit_exact(port):
    src = q8_0_edge_blocks(1 << 14, seed=4)
    got = moe.convert_q8_0_to_q2_0(cuda(src)).cpu().numpy()
    want = port.convert_q8_0_to_q2_0(src)
    diff = (got.reshape(-1, 18) != want.reshape(-1, 18)).any(axis=1)
    assert not diff.any(), f"{int(diff.sum())} of {diff.size} blocks differ, first at {int(np.argmax(diff))}"


def test_unsupported_type_and_shapes_are_rejected():
    z = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    ids = torch.zeros(1, 1, dtype=torch.int32, device="cuda")
    with pytest.raises(moe.FrxError, match="only Q2_0"):
        moe.gemv.moe_q(8, z, None, z, ids, 512, 4, 144 * 4, False)
    with pytest.raises(moe.FrxError, match="multiple of 128"):
        moe.gemv.moe_q(Q2_0, z, None, z, ids, 192, 4, 54 * 4, False)
