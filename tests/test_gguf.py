"""The GGUF reader (frx_gguf_*) on synthetic files written from the published container format:
directory, metadata and offsets on the CPU; the expert loader into the device arena on a GPU,
byte-exact against the oracle's repack."""
import os

import numpy as np
import pytest

from flashrt_b200 import moe, synth
from flashrt_b200.lib import FrxError


def _file(tmp_path, alignment=32, version=3):
    rng = np.random.default_rng(1)
    tensors = [("token_embd.weight", [64, 10], 30, rng.integers(0, 256, 64 * 10 * 2, dtype=np.uint8)),
               ("blk.0.ffn_gate_exps.weight", [128, 128, 4], 42, rng.integers(0, 256, 4 * 128 * 2 * 18, dtype=np.uint8)),
               ("output_norm.weight", [64], 0, rng.integers(0, 256, 64 * 4, dtype=np.uint8))]
    meta = {"general.architecture": "qwen4exp", "qwen4exp.block_count": 48, "qwen4exp.expert_count": 512, "general.file_type": -3,
            "tokenizer.ggml.tokens": ["a", "bc", "def"], "tokenizer.ggml.scores": [1, 2, 3], "qwen4exp.rope.scale": 0.5,
            "general.flag": True}
    path = str(tmp_path / "m.gguf")
    offs = synth.write_gguf(path, meta, tensors, alignment=alignment, version=version)
    return path, tensors, offs


@pytest.mark.parametrize("alignment,version", [(32, 3), (64, 2), (4096, 3)])
def test_directory_and_metadata(tmp_path, alignment, version):
    path, tensors, offs = _file(tmp_path, alignment, version)
    g = moe.Gguf(path)
    assert g.tensor_names() == [t[0] for t in tensors]
    assert g.get_int("qwen4exp.block_count") == 48 and g.get_int("qwen4exp.expert_count") == 512
    assert g.get_int("general.file_type") == -3 and g.get_int("general.flag") == 1
    assert g.get_int("no.such.key", 7) == 7 and g.get_int("general.architecture", 9) == 9   # strings are not integers
    raw = open(path, "rb").read()
    for name, dims, typ, data in tensors:
        t = g.tensor(name)
        assert t["type"] == typ and t["dims"] == dims and t["offset"] == offs[name] and t["offset"] % alignment == 0
        assert t["bytes"] == data.size
        assert raw[t["offset"]:t["offset"] + t["bytes"]] == data.tobytes()
    with pytest.raises(FrxError):
        g.tensor("blk.9.missing")
    g.close()


def test_malformed_files_are_rejected(tmp_path):
    path, _, _ = _file(tmp_path)
    raw = open(path, "rb").read()
    bad = tmp_path / "bad.gguf"
    bad.write_bytes(b"GGML" + raw[4:])
    with pytest.raises(FrxError):
        moe.Gguf(str(bad))
    bad.write_bytes(raw[:100])          # cut inside the metadata
    with pytest.raises(FrxError):
        moe.Gguf(str(bad))
    bad.write_bytes(raw[:len(raw) - 50])  # the last tensor reaches beyond the end
    with pytest.raises(FrxError):
        moe.Gguf(str(bad))
    with pytest.raises(FrxError):
        moe.Gguf(str(tmp_path / "absent.gguf"))


@pytest.mark.gpu
def test_expert_loader_fills_the_arena(tmp_path, port):
    import torch
    n, ff, E, L = 256, 128, 70, 2          # 70 experts: a full piece of 64 and a ragged one
    rng = np.random.default_rng(2)
    tensors, want = [], {}
    for l in range(L):
        mats = [synth.expert_ggml(rng, n, ff) for _ in range(E)]
        for k, nm in enumerate(("ffn_gate_exps", "ffn_up_exps", "ffn_down_exps")):
            dims = [n, ff, E] if k < 2 else [ff, n, E]
            tensors.append((f"blk.{l}.{nm}.weight", dims, 42, np.concatenate([m[k].reshape(-1) for m in mats])))
        for e in range(E):
            want[(l, e)] = port.repack_expert(*mats[e], n, ff)
    tensors.insert(1, ("blk.0.attn_q.weight", [n, n], 30, rng.integers(0, 256, n * n * 2, dtype=np.uint8)))   # something in between
    path = str(tmp_path / "experts.gguf")
    synth.write_gguf(path, {"general.architecture": "qwen4exp"}, tensors)
    g = moe.Gguf(path)
    arena = moe.ExpertArena(L, E, n, ff)
    nbytes, secs = moe.arena_load_gguf(arena, g, 0, L, E)
    assert nbytes == L * E * moe.expert_bytes(n, ff) and secs > 0
    for l in range(L):
        back = arena.read_planar(l, 0, E).cpu().numpy()
        for e in range(E):
            assert np.array_equal(back[e], want[(l, e)]), (l, e)
    with pytest.raises(FrxError):   # a layer the file does not have
        moe.arena_load_gguf(arena, g, 1, 2, E)
    g.close()
