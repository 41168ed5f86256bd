"""Shared set-up for the GPU parity tests: seeded experts on the host (planar, via the oracle's
repack) and in device memory (tiled, via libfrx)."""
from __future__ import annotations

import numpy as np
import torch

from flashrt_b200 import moe, synth


class Experts:
    """E seeded experts (+ optionally one shared expert): planar numpy blobs for the oracle and a
    tiled device copy for the kernels."""

    def __init__(self, port, n, ff, E, seed=synth.SEED_WEIGHTS, shared=True, direct=False):
        self.n, self.ff, self.E = n, ff, E
        rng = np.random.default_rng(seed)
        total = E + (1 if shared else 0)
        if direct:   # drawn in the planar layout directly (large cases)
            self.planar = synth.planar_experts_random(rng, total, n, ff)
        else:
            self.planar = np.stack([port.repack_expert(*synth.expert_ggml(rng, n, ff), n, ff) for _ in range(total)])
        self.blob_bytes = self.planar.shape[1]
        self.stride = moe.expert_stride(n, ff)
        dev = torch.from_numpy(self.planar.reshape(-1)).cuda()
        self.tiled = moe.tile_experts(dev, n, ff, total)
        torch.cuda.synchronize()
        self.base = self.tiled.data_ptr()
        self.shared_ptr = self.base + E * self.stride if shared else None
        self.shared_planar = self.planar[E] if shared else None

    def routed_planar(self):
        return self.planar[:self.E]


def rel_max(a: np.ndarray, b: np.ndarray) -> float:
    """max |a - b| over the RMS of b: the reference's error measure (tests/test_q2_0.cpp:117-124)."""
    rms = float(np.sqrt(np.mean(b.astype(np.float64) ** 2)))
    return float(np.abs(a.astype(np.float64) - b.astype(np.float64)).max() / max(rms, 1e-30))


def cuda(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()
