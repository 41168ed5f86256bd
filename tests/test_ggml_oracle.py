"""The ggml-layout pieces of the CPU oracle (oracle/ggml_oracle.c): the Q8_0 -> Q2_0 requantizer
bit for bit against the reference's own function (arch/qwen4exp/mtp.cu compiled unmodified, where
that library was built), the Q8_1 quantizer and the Q2_0 x Q8_1 dot against their definitions in
numpy. CPU only."""
import numpy as np
import pytest

from flashrt_b200 import synth


def q8_0_edge_blocks(n: int, seed: int = 1) -> np.ndarray:
    """n pairs of Q8_0 blocks {fp16 d; 32 int8} with the cases that stress the requantizer: zero
    scales, scales below and at fp16's subnormal edge, scales that overflow fp16 when multiplied,
    exact halves after scaling, a single large value, and plain Gaussian codes at many magnitudes."""
    rng = np.random.default_rng(seed)
    out = np.zeros((2 * n, 34), np.uint8)
    d = (np.ldexp(1.0, -rng.integers(0, 20, 2 * n)) * 0.01).astype(np.float32)
    kind = np.arange(2 * n) % 89
    d[kind == 0] = 0.0
    d[kind == 1] = 3e-8
    d[kind == 2] = 6e-8
    d[kind == 3] = 60000.0
    out[:, 0:2] = d.astype(np.float16).view(np.uint8).reshape(-1, 2)
    q = np.clip(np.rint(rng.normal(0, 40, (2 * n, 32))), -127, 127).astype(np.int8)
    single = np.arange(2 * n) % 13 == 5
    q[single] = 0
    q[single, 0] = 127
    halves = np.arange(2 * n) % 11 == 7
    q[halves] = np.where(np.arange(32) % 2 == 1, 64, -64).astype(np.int8)
    out[:, 2:] = q.view(np.uint8)
    return out.reshape(-1)


def test_requantizer_matches_the_reference_function(port):
    from oracle import oracle
    src = q8_0_edge_blocks(1 << 15)
    got = port.convert_q8_0_to_q2_0(src)
    want = oracle.ref_convert_q8_0_to_q2_0(src)
    if want is None:
        pytest.skip("oracle/_ref/libfrx_ref_mtp.so not built (needs the reference tree and nvcc)")
    diff = (got.reshape(-1, 18) != want.reshape(-1, 18)).any(axis=1)
    assert not diff.any(), f"{int(diff.sum())} of {diff.size} blocks differ, first at {int(np.argmax(diff))}"


def test_requantizer_known_blocks(port):
    # all zeros -> scale 0, every code 1 (the value 0); one large value -> that value maps to code 3 (= +2 d) or 2
    z = np.zeros(68, np.uint8)
    out = port.convert_q8_0_to_q2_0(z)
    assert out[0] == 0 and out[1] == 0 and np.all(out[2:] == 0x55)
    one = np.zeros(68, np.uint8)
    one[0:2] = np.frombuffer(np.float16(0.5).tobytes(), np.uint8)
    one[34:36] = one[0:2]
    one[2] = 100
    out = port.convert_q8_0_to_q2_0(one)
    d = np.frombuffer(out[0:2].tobytes(), np.float16)[0]
    assert d > 0
    code0 = out[2] & 3
    assert code0 in (2, 3) and abs((code0 - 1) * float(d) - 50.0) <= 0.5 * float(d) + 1e-3
    rest = np.unpackbits(out[2:].reshape(-1, 1), axis=1, bitorder="little").reshape(-1, 4, 2)
    codes = rest[:, :, 0] + 2 * rest[:, :, 1]
    assert np.all(codes.reshape(-1)[1:] == 1)


def test_q8_1_and_dot_follow_their_definitions(port):
    rng = np.random.default_rng(3)
    ncols, nrows = 640, 5                      # 640 pads to 1024 values per activation row
    x = rng.standard_normal((2, ncols)).astype(np.float32)
    x[1, 64:96] = 0.0                          # an all-zero block: d = 0, codes 0
    xq = port.quantize_q8_1(x)
    assert xq.shape == (2, 1024 // 32 * 36)
    blocks = xq.reshape(2, -1, 36)
    d = blocks[:, :, 0:2].copy().view(np.float16).astype(np.float32)[:, :, 0]
    q = blocks[:, :, 4:].view(np.int8).astype(np.int32)
    xp = np.zeros((2, 1024), np.float32)
    xp[:, :ncols] = x
    xb = xp.reshape(2, -1, 32)
    amax = np.abs(xb).max(axis=2)
    assert np.array_equal(d, (amax / np.float32(127.0)).astype(np.float16).astype(np.float32))
    with np.errstate(invalid="ignore", divide="ignore"):
        want_q = np.where(amax[:, :, None] == 0, 0, np.sign(xb) * np.floor(np.abs(xb / (amax / np.float32(127.0))[:, :, None]) + 0.5))
    assert np.array_equal(q, want_q.astype(np.int32))
    assert np.all(q[:, ncols // 32:] == 0) and np.all(d[:, ncols // 32:] == 0)
    # the dot: dequantised weights times dequantised activations, to float rounding
    w = synth.ggml_blocks(rng, nrows, ncols)
    wf = port.dequant_ggml(w, nrows, ncols).astype(np.float64)
    af = (q[:, :ncols // 32] * d[:, :ncols // 32, None]).reshape(2, ncols).astype(np.float64)
    ids = np.zeros((2, 1), np.int32)
    got = port.moe_q2_0(w.reshape(-1), None, xq.reshape(-1), ids, ncols, nrows, 0, False)
    want = af @ wf.T
    assert np.abs(got[:, 0, :] - want).max() <= 1e-5 * np.abs(want).max()
