"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configs.

No public dataset or checkpoint is involved: weights are random Q2_0 blocks, activations and
router logits are Gaussian, and skewed routing is a Gumbel-top-k draw from a Zipf law.

  weights      2-bit codes uniform in {0..3}; fp16 block scales |N(0, 0.02)|, exact zeros lifted
               to the smallest normal half; generated as ggml blocks {fp16 d; 16 code bytes}
  activations  fp32 N(0, 1) (optionally rounded through bf16)
  logits       fp32 N(0, 1); or, for Zipf(s) routing, -s * ln(rank(e)) + Gumbel(0, 1) with a
               seeded random rank permutation, whose top-k is sampling without replacement
               with probability proportional to rank^-s
"""
from __future__ import annotations

import numpy as np

SEED_WEIGHTS, SEED_ACT, SEED_LOGITS, SEED_ZIPF = 20260927, 7, 9, 11
BLOCK, BLOCK_BYTES = 64, 18


def ggml_blocks(rng: np.random.Generator, rows: int, cols: int, scale_sd: float = 0.02) -> np.ndarray:
    """rows x cols Q2_0 weights as ggml blocks: uint8 [rows * cols/64][18]."""
    nblk = rows * (cols // BLOCK)
    out = np.empty((nblk, BLOCK_BYTES), np.uint8)
    d = np.abs(rng.standard_normal(nblk, dtype=np.float32) * np.float32(scale_sd)).astype(np.float16)
    d[d == 0] = np.float16(6.103515625e-05)
    out[:, 0:2] = d.view(np.uint8).reshape(nblk, 2)
    out[:, 2:] = rng.integers(0, 256, size=(nblk, 16), dtype=np.uint8)
    return out


def expert_ggml(rng: np.random.Generator, n: int, ff: int, scale_sd: float = 0.02):
    """gate [ff][n], up [ff][n], down [n][ff] as ggml blocks."""
    return ggml_blocks(rng, ff, n, scale_sd), ggml_blocks(rng, ff, n, scale_sd), ggml_blocks(rng, n, ff, scale_sd)


def planar_experts_random(rng: np.random.Generator, n_experts: int, n: int, ff: int, scale_sd: float = 0.02) -> np.ndarray:
    """n_experts planar blobs drawn directly in the planar layout (a permutation of uniform codes
    is uniform): uint8 [n_experts][expert_bytes]."""
    nb_gu, nb_dn = ff * (n // BLOCK), n * (ff // BLOCK)
    blob = 2 * nb_gu * BLOCK_BYTES + nb_dn * BLOCK_BYTES
    out = np.empty((n_experts, blob), np.uint8)
    for e in range(n_experts):
        off = 0
        for nblk in (nb_gu, nb_gu, nb_dn):
            out[e, off:off + nblk * 16] = rng.integers(0, 256, size=nblk * 16, dtype=np.uint8)
            d = np.abs(rng.standard_normal(nblk, dtype=np.float32) * np.float32(scale_sd)).astype(np.float16)
            d[d == 0] = np.float16(6.103515625e-05)
            out[e, off + nblk * 16:off + nblk * 18] = d.view(np.uint8)
            off += nblk * 18
    return out


def activations(T: int, n: int, seed: int = SEED_ACT, through_bf16: bool = False) -> np.ndarray:
    x = np.random.default_rng(seed).standard_normal((T, n), dtype=np.float32)
    if through_bf16:   # round to nearest even on the top 16 bits
        u = x.view(np.uint32)
        u = ((u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000).astype(np.uint32)
        x = u.view(np.float32)
    return x


def router_logits(T: int, E: int, seed: int = SEED_LOGITS) -> np.ndarray:
    return np.random.default_rng(seed).standard_normal((T, E), dtype=np.float32)


def zipf_logits(T: int, E: int, s: float = 1.1, seed: int = SEED_ZIPF) -> np.ndarray:
    rng = np.random.default_rng(seed)
    rank = rng.permutation(E).astype(np.float64) + 1.0
    u = rng.random((T, E))
    gumbel = -np.log(-np.log(np.clip(u, 1e-300, 1.0 - 1e-16)))
    return (-s * np.log(rank)[None, :] + gumbel).astype(np.float32)


def tie_heavy_logits(T: int, E: int, seed: int = 9) -> np.ndarray:
    """Logits rounded to multiples of 0.25 so exact ties are common (the construction of the
    reference's router test, tests/test_route_topk.cpp:24-27)."""
    g = np.random.default_rng(seed).standard_normal((T, E), dtype=np.float32) * np.float32(2.0)
    return (np.round(g * 4.0) / 4.0).astype(np.float32)


def write_gguf(path: str, meta: dict, tensors: list, alignment: int = 32, version: int = 3) -> dict:
    """Writes a GGUF file (the published container format) for tests and examples. meta: key ->
    int (stored as u32, or i64 when negative or large), float (f32), bool, str, or a list of str /
    int (an array). tensors: (name, dims fastest first, ggml type id, uint8 data) in file order.
    Returns name -> absolute file offset of the tensor's data."""
    import struct

    def gstr(s: str) -> bytes:
        b = s.encode()
        return struct.pack("<Q", len(b)) + b

    def value(v) -> bytes:
        if isinstance(v, bool):
            return struct.pack("<IB", 7, int(v))
        if isinstance(v, int):
            return struct.pack("<II", 4, v) if 0 <= v < 2 ** 32 else struct.pack("<Iq", 11, v)
        if isinstance(v, float):
            return struct.pack("<If", 6, v)
        if isinstance(v, str):
            return struct.pack("<I", 8) + gstr(v)
        if isinstance(v, list):
            if all(isinstance(x, str) for x in v):
                return struct.pack("<IIQ", 9, 8, len(v)) + b"".join(gstr(x) for x in v)
            return struct.pack("<IIQ", 9, 5, len(v)) + b"".join(struct.pack("<i", x) for x in v)
        raise TypeError(type(v))

    meta = dict(meta)
    if alignment != 32:
        meta["general.alignment"] = alignment
    head = struct.pack("<IIQQ", 0x46554747, version, len(tensors), len(meta))
    for k, v in meta.items():
        head += gstr(k) + value(v)
    rel, at = {}, 0
    for name, dims, typ, data in tensors:
        at = (at + alignment - 1) // alignment * alignment
        rel[name] = at
        head += gstr(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims) + struct.pack("<IQ", typ, at)
        at += data.size
    data_start = (len(head) + alignment - 1) // alignment * alignment
    with open(path, "wb") as f:
        f.write(head)
        f.write(b"\0" * (data_start - len(head)))
        pos = 0
        for name, dims, typ, data in tensors:
            f.write(b"\0" * (rel[name] - pos))
            f.write(np.ascontiguousarray(data).tobytes())
            pos = rel[name] + data.size
    return {name: data_start + off for name, off in rel.items()}
