"""Generates tests/golden/q2moe_small.npz from the reference's own CPU sources.

Run where oracle/_ref/libfrx_ref.so exists (it is compiled from the reference tree by
oracle/Makefile):  python tests/golden/make_golden.py

Inputs are seeded; every output is computed by the reference code (its scalar path for the
bit-exact vectors, its AVX-512 moe_cpu for the layer output). The fixture lets the oracle and the
CUDA path be checked against reference results on machines that do not have the reference.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from flashrt_b200 import synth  # noqa: E402
from oracle import oracle  # noqa: E402


def main():
    ref = oracle.ref()
    if ref is None:
        raise SystemExit("oracle/_ref/libfrx_ref.so is missing: run `make -C oracle` where the reference tree is")
    n, ff, E, K, T = 256, 128, 8, 3, 5
    rng = np.random.default_rng(synth.SEED_WEIGHTS)
    ggml = [synth.expert_ggml(rng, n, ff) for _ in range(E)]
    planar = np.stack([ref.repack_expert(g, u, d, n, ff) for g, u, d in ggml])
    x = synth.activations(T, n)
    logits = synth.router_logits(T, E)
    xq = np.stack([ref.quantize_q8(x[t])[0] for t in range(T)])
    xd = np.stack([ref.quantize_q8(x[t])[1] for t in range(T)])
    gate_rows = np.stack([ref.matvec(planar[e, :ref.mat_bytes(ff, n)], ff, n, x[0], avx=False) for e in range(E)])
    ffn = np.stack([ref.expert_ffn(planar[e], n, ff, x[:4], avx=False) for e in range(E)])   # [E][4][n], scalar path
    # routing for the layer output: top-K of the logits by a stable sort (what the reference's router does)
    ids = np.argsort(-logits, axis=1, kind="stable")[:, :K].astype(np.int32)
    p = np.exp(logits - logits.max(1, keepdims=True))
    p = p / p.sum(1, keepdims=True)
    sel = np.take_along_axis(p, ids, 1)
    wts = (sel / sel.sum(1, keepdims=True)).astype(np.float32)
    moe = ref.moe_cpu(planar, planar.shape[1], E, n, ff, x, ids, wts, workers=2)
    np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "q2moe_small.npz"),
                        shape=np.array([n, ff, E, K, T], np.int32),
                        ggml_gate=np.stack([g for g, _, _ in ggml]), ggml_up=np.stack([u for _, u, _ in ggml]),
                        ggml_down=np.stack([d for _, _, d in ggml]), planar=planar, x=x, logits=logits, xq=xq, xd=xd,
                        gate_rows_tok0=gate_rows, expert_ffn_scalar=ffn, ids=ids, wts=wts, moe_cpu_out=moe,
                        moe_cpu_avx512=np.array([int(ref.have_avx512())], np.int32))
    print("wrote q2moe_small.npz")


if __name__ == "__main__":
    main()
