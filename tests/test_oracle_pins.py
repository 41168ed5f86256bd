"""The scalar oracle against the reference's own known answers and algebraic identities
(the pins of the reference's tests/test_q2_0.cpp and tests/test_moe_cpu.cpp). CPU only."""
import numpy as np

from flashrt_b200 import synth


def test_fp16_known_values(port):
    # tests/test_q2_0.cpp:69-71
    assert port.fp32_to_fp16(1.0) == 0x3C00
    assert port.fp32_to_fp16(-2.0) == 0xC000
    assert port.fp32_to_fp16(65504.0) == 0x7BFF
    assert port.fp16_to_fp32(0x3555) == 0.333251953125
    assert port.fp16_to_fp32(0x0001) == 5.960464477539063e-08


def test_fp16_matches_ieee_everywhere(port):
    # every half value converts exactly as IEEE (numpy) does, and round-trips
    h = np.arange(0x7C00, dtype=np.uint16)   # all finite non-negative halves
    ieee = h.view(np.float16).astype(np.float32)
    for i in range(0, len(h), 97):
        assert port.fp16_to_fp32(int(h[i])) == float(ieee[i])
        assert port.fp32_to_fp16(float(ieee[i])) == int(h[i])
    rng = np.random.default_rng(1)
    f = (rng.standard_normal(4000).astype(np.float32) * np.float32(10.0) ** rng.integers(-9, 5, 4000)).astype(np.float32)
    want = f.astype(np.float16).view(np.uint16)
    got = np.array([port.fp32_to_fp16(float(v)) for v in f], np.uint16)
    assert np.array_equal(got, want)


def test_expert_blob_size(port):
    # tests/test_q2_0.cpp:141 and the benchmark shape
    assert port.expert_bytes(2560, 640) == 1382400
    assert port.expert_bytes(2048, 512) == 884736
    assert port.mat_bytes(512, 2048) == 294912


def test_repack_is_elementwise_placement(port):
    # tests/test_q2_0.cpp:74-86
    rng = np.random.default_rng(20260927)
    rows, cols = 8, 4096
    g = synth.ggml_blocks(rng, rows, cols)
    packed = port.repack(g, rows, cols)
    nblk = g.shape[0]
    codes = packed[:nblk * 16].reshape(nblk, 16)
    scales = packed[nblk * 16:].reshape(nblk, 2)
    j = np.arange(64)
    q = (g[:, 2 + j // 4] >> (2 * (j % 4))) & 3                      # [nblk][64] element codes
    want = np.zeros((nblk, 16), np.uint8)
    for e in range(64):
        want[:, e % 16] |= (q[:, e] << (2 * (e // 16))).astype(np.uint8)
    assert np.array_equal(codes, want)
    assert np.array_equal(scales, g[:, :2])


def test_matvec_equals_ggml_dot(port):
    # tests/test_q2_0.cpp:99-109: max abs diff 0
    rng = np.random.default_rng(20260927)
    for rows, cols in ((96, 2560), (160, 640), (64, 2048)):
        g = synth.ggml_blocks(rng, rows, cols)
        packed = port.repack(g, rows, cols)
        x = rng.standard_normal(cols, dtype=np.float32)
        q, d = port.quantize_q8(x)
        y = port.matvec(packed, rows, cols, q, d)
        row_bytes = (cols // 64) * 18
        for r in range(rows):
            assert y[r] == port.dot_ggml(g.reshape(-1)[r * row_bytes:(r + 1) * row_bytes], cols, q, d)


def test_matvec_row_range_touches_only_its_rows(port):
    # tests/test_q2_0.cpp:129-133
    rng = np.random.default_rng(3)
    g = synth.ggml_blocks(rng, 32, 256)
    packed = port.repack(g, 32, 256)
    q, d = port.quantize_q8(rng.standard_normal(256, dtype=np.float32))
    full = port.matvec(packed, 32, 256, q, d)
    part = port.matvec(packed, 32, 256, q, d, 10, 20)
    assert np.array_equal(part, full[10:20])


def test_quantize_q8_definition(port):
    rng = np.random.default_rng(5)
    x = rng.standard_normal(256, dtype=np.float32)
    x[32:64] = 0.0                       # an all-zero block: scale 0, codes 0
    x[64] = 2.5 * np.abs(x[64:96]).max() # a clear maximum
    q, d = port.quantize_q8(x)
    assert np.all(q[32:64] == 0) and d[1] == 0.0
    for b in range(8):
        blk = x[32 * b:32 * b + 32]
        dd = np.float32(np.abs(blk).max()) / np.float32(127.0)
        assert d[b] == np.float32(np.float16(dd))
        if dd != 0:
            idv = np.float32(1.0) / dd
            v = blk * idv
            want = np.where(v >= 0, np.floor(v + np.float32(0.5)), np.ceil(v - np.float32(0.5)))   # half away from zero
            # floor(v + 0.5) equals roundf except when v + 0.5 rounds up in float; compare loosely then exactly on safe values
            safe = np.abs(np.abs(v - np.trunc(v)) - 0.5) > 1e-3
            assert np.array_equal(q[32 * b:32 * b + 32][safe], want[safe].astype(np.int8))
    assert np.abs(q).max() == 127


def test_expert_vs_fp32_swiglu(port):
    # tests/test_q2_0.cpp:147-181: the Q8 error of the whole expert is below 5 % rel L2
    rng = np.random.default_rng(20260927)
    n, ff = 512, 256
    g, u, dn = synth.expert_ggml(rng, n, ff, 0.01)
    blob = port.repack_expert(g, u, dn, n, ff)
    x = rng.standard_normal(n, dtype=np.float32)
    q, d = port.quantize_q8(x)
    out = port.expert_ffn(blob, n, ff, q, d)
    wg, wu, wd = port.dequant_ggml(g, ff, n).astype(np.float64), port.dequant_ggml(u, ff, n).astype(np.float64), port.dequant_ggml(dn, n, ff).astype(np.float64)
    gs, us = wg @ x, wu @ x
    h = gs / (1 + np.exp(-gs)) * us
    o = wd @ h
    rel = np.linalg.norm(out - o) / np.linalg.norm(o)
    assert rel < 0.05


def test_dequant_planar_equals_ggml(port):
    rng = np.random.default_rng(8)
    g = synth.ggml_blocks(rng, 16, 512)
    assert np.array_equal(port.dequant_planar(port.repack(g, 16, 512), 16, 512), port.dequant_ggml(g, 16, 512))


def test_moe_layer_is_weighted_sum_of_experts(port):
    # tests/test_moe_cpu.cpp:66-85: the layer equals a loop of expert_ffn calls, weighted, summed in expert order
    rng = np.random.default_rng(11)
    n, ff, E, K, T = 256, 128, 6, 3, 3
    blobs = np.stack([port.repack_expert(*synth.expert_ggml(rng, n, ff), n, ff) for _ in range(E)])
    x = rng.standard_normal((T, n), dtype=np.float32)
    ids = np.array([[4, 0, 2], [1, 5, 3], [2, 1, 0]], np.int32)
    wts = rng.random((T, K), dtype=np.float32)
    out, ys, _ = port.moe_layer(blobs, blobs.shape[1], None, n, ff, x, ids, wts, want_slots=True)
    xq, xd = port.quantize_q8(x)
    for t in range(T):
        acc = np.zeros(n, np.float32)
        for k in np.argsort(ids[t]):
            y = port.expert_ffn(blobs[ids[t, k]], n, ff, xq[t], xd[t])
            assert np.array_equal(y, ys[t * K + k])
            acc = acc + wts[t, k] * y
        assert np.array_equal(acc, out[t])
    # threads do not change the result
    assert np.array_equal(out, port.moe_layer(blobs, blobs.shape[1], None, n, ff, x, ids, wts, n_threads=4))


def test_route_ties_and_weights(port):
    # tests/test_route_topk.cpp:24-69: ids equal a stable sort by logit; weights within 1e-5 of a double reference
    T, E, K = 256, 512, 10
    lg = synth.tie_heavy_logits(T, E)
    ids, wts, _ = port.route(lg, K)
    for t in range(T):
        order = np.argsort(-lg[t], kind="stable")[:K]
        assert np.array_equal(ids[t], order)
        p = np.exp(lg[t].astype(np.float64) - lg[t].max())
        p /= p.sum()
        assert np.abs(wts[t] - p[order] / p[order].sum()).max() < 1e-5


def test_router_projection_restatement_widens_bf16_exactly():
    # bf16 -> fp32 is a 16-bit shift; the restatement's float64 sum against torch's own widening
    import torch
    from oracle import oracle
    rng = np.random.default_rng(5)
    w = torch.from_numpy(rng.standard_normal((9, 256), dtype=np.float32)).to(torch.bfloat16)
    x = rng.standard_normal((3, 256), dtype=np.float32)
    got = oracle.router_logits(w.view(torch.int16).numpy().view(np.uint16), x)
    want = x.astype(np.float64) @ w.to(torch.float64).numpy().T
    assert np.array_equal(got, want)
