"""The scalar oracle against the reference's own CPU sources compiled unmodified (oracle/_ref),
on seeded inputs. Scalar-vs-scalar comparisons are bit for bit; comparisons with the reference's
AVX-512 kernel use the reference's own tolerances (tests/test_q2_0.cpp:114-127,178-181;
tests/test_moe_cpu.cpp:79-84). CPU only; skipped where the reference library was not built."""
import numpy as np

from flashrt_b200 import synth


def test_fp16_same(port, ref):
    for h in list(range(0, 0x7C00, 31)) + [0x0001, 0x03FF, 0x0400, 0x7BFF, 0x8001, 0xFBFF]:
        assert port.fp16_to_fp32(h) == ref.fp16_to_fp32(h)
    rng = np.random.default_rng(2)
    for v in (rng.standard_normal(3000) * 10.0 ** rng.integers(-9, 6, 3000)).astype(np.float32):
        assert port.fp32_to_fp16(float(v)) == ref.fp32_to_fp16(float(v))


def test_sizes_same(port, ref):
    for n, ff in ((2560, 640), (2048, 512), (256, 128)):
        assert port.expert_bytes(n, ff) == ref.expert_bytes(n, ff)
        assert port.mat_bytes(ff, n) == ref.mat_bytes(ff, n)


def test_repack_same(port, ref):
    rng = np.random.default_rng(20260927)
    n, ff = 512, 256
    g, u, d = synth.expert_ggml(rng, n, ff)
    assert np.array_equal(port.repack(g, ff, n), ref.repack(g, ff, n))
    assert np.array_equal(port.repack_expert(g, u, d, n, ff), ref.repack_expert(g, u, d, n, ff))


def test_quantize_q8_same(port, ref):
    rng = np.random.default_rng(7)
    for scale in (1.0, 1e-3, 50.0):
        x = (rng.standard_normal(2048) * scale).astype(np.float32)
        x[100:132] = 0
        q, d = port.quantize_q8(x)
        rq, rd = ref.quantize_q8(x)
        assert np.array_equal(q, rq) and np.array_equal(d, rd)


def test_matvec_scalar_bit_exact_and_avx_close(port, ref):
    rng = np.random.default_rng(20260927)
    for rows, cols in ((96, 2560), (160, 640), (128, 2048)):
        g = synth.ggml_blocks(rng, rows, cols)
        packed = port.repack(g, rows, cols)
        x = rng.standard_normal(cols, dtype=np.float32)
        q, d = port.quantize_q8(x)
        y = port.matvec(packed, rows, cols, q, d)
        assert np.array_equal(y, ref.matvec(packed, rows, cols, x, avx=False))
        row = (cols // 64) * 18
        assert port.dot_ggml(g.reshape(-1)[:row], cols, q, d) == ref.dot_ggml(g.reshape(-1)[:row], cols, x)
        if ref.have_avx512():
            ya = ref.matvec(packed, rows, cols, x, avx=True)
            assert np.abs(ya - y).max() / np.sqrt(np.mean(y.astype(np.float64) ** 2)) < 1e-5


def test_expert_ffn_scalar_bit_exact(port, ref):
    rng = np.random.default_rng(20260927)
    for n, ff in ((512, 256), (2048, 512)):
        blob = port.repack_expert(*synth.expert_ggml(rng, n, ff), n, ff)
        x = rng.standard_normal((3, n), dtype=np.float32)
        xq, xd = port.quantize_q8(x)
        want = ref.expert_ffn(blob, n, ff, x, avx=False)
        for t in range(3):
            assert np.array_equal(port.expert_ffn(blob, n, ff, xq[t], xd[t]), want[t])
        if ref.have_avx512():
            avx = ref.expert_ffn(blob, n, ff, x, avx=True)
            assert np.linalg.norm(avx - want) / np.linalg.norm(want) < 1e-4


def test_moe_layer_vs_moe_cpu(port, ref):
    # moe_cpu picks the AVX-512 kernel when the CPU has it, so this is a tolerance check
    # (rel L2 < 1e-5 is the reference's own bound for moe_cpu against an expert_ffn loop).
    rng = np.random.default_rng(11)
    n, ff, E, K, T = 512, 256, 16, 4, 9
    blobs = np.stack([port.repack_expert(*synth.expert_ggml(rng, n, ff), n, ff) for _ in range(E)])
    x = rng.standard_normal((T, n), dtype=np.float32)
    ids, wts, _ = port.route(synth.router_logits(T, E), K)
    out = port.moe_layer(blobs, blobs.shape[1], None, n, ff, x, ids, wts)
    for workers in (1, 3):
        got = ref.moe_cpu(blobs, blobs.shape[1], E, n, ff, x, ids, wts, workers=workers)
        rel = np.linalg.norm(got - out) / np.linalg.norm(out)
        assert rel < (1e-5 if ref.have_avx512() else 1e-12)
    if not ref.have_avx512():
        assert np.array_equal(got, out)
