"""Router top-k and the Q8 activation quantizer on the GPU against the oracle: ids, counts and
int8 codes bit-exact; weights within 1e-6 of the oracle and 1e-5 of a double reference. Needs a GPU."""
import numpy as np
import pytest
import torch

from flashrt_b200 import moe, synth
from helpers import cuda

pytestmark = pytest.mark.gpu


def test_route_tie_heavy_full_size():
    # the reference's own router test (tests/test_route_topk.cpp): 16,384 tokens, 512 experts,
    # top-10, logits rounded to 0.25 so exact ties are common
    T, E, K = 16384, 512, 10
    lg = synth.tie_heavy_logits(T, E)
    counts = torch.zeros(E, dtype=torch.int32, device="cuda")
    tail = torch.zeros(E, dtype=torch.int32, device="cuda")
    ids, wts = moe.moe_route_topk(cuda(lg), K, counts=counts, tail_counts=tail, tail_from=T - 100)
    ids, wts = ids.cpu().numpy(), wts.cpu().numpy()
    order = np.argsort(-lg, axis=1, kind="stable")[:, :K]
    assert np.array_equal(ids, order)
    assert np.array_equal(counts.cpu().numpy(), np.bincount(order.reshape(-1), minlength=E))
    assert np.array_equal(tail.cpu().numpy(), np.bincount(order[T - 100:].reshape(-1), minlength=E))
    l64 = lg.astype(np.float64)
    p = np.exp(l64 - l64.max(1, keepdims=True))
    p /= p.sum(1, keepdims=True)
    sel = np.take_along_axis(p, order, 1)
    assert np.abs(wts - sel / sel.sum(1, keepdims=True)).max() < 1e-5


@pytest.mark.parametrize("T,E,K", [(1, 512, 10), (64, 512, 10), (777, 512, 10), (33, 128, 8), (40, 1000, 32), (9, 8, 3), (5, 40, 32)])
def test_route_matches_oracle(port, T, E, K):
    lg = synth.router_logits(T, E)
    ids, wts = moe.moe_route_topk(cuda(lg), K)
    oid, ow, _ = port.route(lg, K)
    assert np.array_equal(ids.cpu().numpy(), oid)
    assert np.abs(wts.cpu().numpy() - ow).max() < 1e-6


def test_route_zipf_and_signed_zero(port):
    lg = synth.zipf_logits(512, 512)
    ids, wts = moe.moe_route_topk(cuda(lg), 10)
    oid, ow, _ = port.route(lg, 10)
    assert np.array_equal(ids.cpu().numpy(), oid)
    assert np.abs(wts.cpu().numpy() - ow).max() < 1e-6
    z = np.zeros((2, 64), np.float32)
    z[0, ::2] = -0.0                     # -0.0 and +0.0 tie: lower index first
    z[1, 5] = -np.inf
    ids, _ = moe.moe_route_topk(cuda(z), 4)
    assert np.array_equal(ids.cpu().numpy(), np.array([[0, 1, 2, 3], [0, 1, 2, 3]]))


def test_route_rejects_unsupported_shapes():
    lg = torch.zeros(4, 2048, device="cuda")
    with pytest.raises(moe.FrxError, match="unsupported shape"):
        moe.moe_route_topk(lg, 10)


def test_quantize_q8_bit_exact(port):
    rng = np.random.default_rng(7)
    x = rng.standard_normal((37, 2048), dtype=np.float32)
    x[1] *= 1e-6
    x[2] *= 3e4
    x[3, 64:96] = 0.0
    x[4, :32] = np.arange(-16, 16, dtype=np.float32) + 0.5          # amax 15.5
    x[5, :32] = 0
    x[5, 0], x[5, 1], x[5, 2], x[5, 3] = 127.0, 2.5, -2.5, 0.5       # d = 1: exact halves round away from zero
    x[6, :32] = 1e-30                                               # scale underflows in fp16
    q, d = moe.quantize_q8(cuda(x))
    oq, od = port.quantize_q8(x)
    assert np.array_equal(q.cpu().numpy(), oq)
    assert np.array_equal(d.cpu().numpy(), od)
    assert list(oq[5, :4]) == [127, 3, -3, 1]
    # the same rows from a buffer that is only 4-byte aligned (the one-value-per-lane form of the kernel)
    buf = torch.empty(x.size + 1, device="cuda")
    shifted = buf[1:].view(x.shape)
    shifted.copy_(cuda(x))
    assert shifted.data_ptr() % 16 == 4
    q2, d2 = moe.quantize_q8(shifted)
    assert torch.equal(q2, q) and torch.equal(d2, d)


def test_quantize_q8_empty_and_bad_shape():
    q, d = moe.quantize_q8(torch.zeros(0, 256, device="cuda"))
    assert q.shape == (0, 256)
    with pytest.raises(moe.FrxError):
        moe.quantize_q8(torch.zeros(2, 48, device="cuda"))


@pytest.mark.parametrize("T,E,n,gate", [(1, 512, 2048, True), (64, 512, 2048, True), (7, 33, 512, False), (200, 128, 1024, True)])
def test_router_projection(T, E, n, gate):
    # logits = W_r x (bf16 weights, fp32 activations and sums) and the shared expert's gate logit
    # in the same launch; tolerance against a float64 sum: fp32 accumulation over n terms
    from oracle import oracle
    rng = np.random.default_rng(3)
    w = torch.from_numpy(rng.standard_normal((E, n), dtype=np.float32) * 0.05).to(torch.bfloat16)
    wg = torch.from_numpy(rng.standard_normal(n, dtype=np.float32) * 0.05).to(torch.bfloat16) if gate else None
    x = rng.standard_normal((T, n), dtype=np.float32)
    logits, g = moe.router_logits(w.cuda(), wg.cuda() if gate else None, cuda(x))
    want = oracle.router_logits(w.view(torch.int16).numpy().view(np.uint16), x)
    scale = np.abs(want).max()
    assert np.abs(logits.cpu().numpy() - want).max() < 2e-6 * scale * np.sqrt(n / 256)
    if gate:
        wantg = oracle.router_logits(wg.view(torch.int16).numpy().view(np.uint16)[None, :], x)[:, 0]
        assert np.abs(g.cpu().numpy() - wantg).max() < 2e-6 * max(scale, np.abs(wantg).max()) * np.sqrt(n / 256)
    # feeding the router: the ids of the GPU logits are the ids of their own values
    ids, _ = moe.moe_route_topk(logits, min(8, E))
    top = np.argsort(-logits.cpu().numpy(), axis=1, kind="stable")[:, :min(8, E)]
    assert np.array_equal(ids.cpu().numpy(), top)
