"""The scalar oracle against the committed fixture, whose outputs were computed by the reference's
own CPU code (tests/golden/make_golden.py). CPU only."""
import os

import numpy as np
import pytest

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "q2moe_small.npz")


@pytest.fixture(scope="module")
def gold():
    return np.load(GOLD)


def test_repack_matches_reference(port, gold):
    n, ff, E, K, T = (int(v) for v in gold["shape"])
    for e in range(E):
        assert np.array_equal(port.repack_expert(gold["ggml_gate"][e], gold["ggml_up"][e], gold["ggml_down"][e], n, ff),
                              gold["planar"][e])


def test_q8_matches_reference(port, gold):
    q, d = port.quantize_q8(gold["x"])
    assert np.array_equal(q, gold["xq"]) and np.array_equal(d, gold["xd"])


def test_matvec_matches_reference_scalar(port, gold):
    n, ff, E, K, T = (int(v) for v in gold["shape"])
    for e in range(E):
        y = port.matvec(gold["planar"][e][:port.mat_bytes(ff, n)], ff, n, gold["xq"][0], gold["xd"][0])
        assert np.array_equal(y, gold["gate_rows_tok0"][e])


def test_expert_ffn_matches_reference_scalar(port, gold):
    n, ff, E, K, T = (int(v) for v in gold["shape"])
    for e in range(E):
        for t in range(4):
            assert np.array_equal(port.expert_ffn(gold["planar"][e], n, ff, gold["xq"][t], gold["xd"][t]),
                                  gold["expert_ffn_scalar"][e][t])


def test_route_matches_fixture(port, gold):
    n, ff, E, K, T = (int(v) for v in gold["shape"])
    ids, wts, _ = port.route(gold["logits"], int(K))
    assert np.array_equal(ids, gold["ids"])
    assert np.abs(wts - gold["wts"]).max() < 1e-6


def test_layer_matches_reference_moe_cpu(port, gold):
    n, ff, E, K, T = (int(v) for v in gold["shape"])
    out = port.moe_layer(gold["planar"], gold["planar"].shape[1], None, int(n), int(ff), gold["x"], gold["ids"], gold["wts"])
    ref = gold["moe_cpu_out"]
    if gold["moe_cpu_avx512"][0]:   # the reference summed with its AVX-512 kernel: its own 1e-5 bound
        assert np.linalg.norm(out - ref) / np.linalg.norm(ref) < 1e-5
    else:
        assert np.array_equal(out, ref)
