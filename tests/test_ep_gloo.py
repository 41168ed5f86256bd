"""Expert-parallel composition on CPU: two gloo ranks each sum the experts they hold (computed by
the CPU oracle, standing in for the kernels), all-reduce, and must reproduce the full layer. This
covers the host-side partition and exchange logic of flashrt_b200.ep without a GPU."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port_no, ret):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port_no)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from flashrt_b200 import synth
    from flashrt_b200.ep import expert_range
    from oracle import oracle
    port = oracle.port()
    n, ff, E, K, T = 256, 128, 10, 3, 6
    rng = np.random.default_rng(synth.SEED_WEIGHTS)
    planar = np.stack([port.repack_expert(*synth.expert_ggml(rng, n, ff), n, ff) for _ in range(E)])
    x = synth.activations(T, n)
    ids, wts, _ = port.route(synth.router_logits(T, E), K)
    lo, hi = expert_range(rank, world, E)
    _, ys, _ = port.moe_layer(planar, planar.shape[1], None, n, ff, x, ids, wts, want_slots=True)
    part = np.zeros((T, n), np.float32)
    for t in range(T):
        for k in np.argsort(ids[t]):
            if lo <= ids[t, k] < hi:
                part[t] = part[t] + wts[t, k] * ys[t * K + k]
    tot = torch.from_numpy(part.copy())
    dist.all_reduce(tot)
    full = port.moe_layer(planar, planar.shape[1], None, n, ff, x, ids, wts)
    err = float(np.abs(tot.numpy() - full).max() / np.sqrt(np.mean(full.astype(np.float64) ** 2)))
    # with a shared expert dealt among the ranks by token ranges: every rank adds the shared expert's
    # gated output for its own tokens only, and the sum of the parts is the full layer again
    from flashrt_b200.ep import shared_token_range
    shared_blob = port.repack_expert(*synth.expert_ggml(rng, n, ff), n, ff)
    gate = np.linspace(-1.0, 1.0, T).astype(np.float32)
    full_sh, _, ysh = port.moe_layer(planar, planar.shape[1], shared_blob, n, ff, x, ids, wts, gate, want_slots=True)
    t0, t1 = shared_token_range(rank, world, T)
    part_sh = part.copy()
    sig = 1.0 / (1.0 + np.exp(-gate.astype(np.float64)))
    for t in range(t0, t1):
        part_sh[t] = part_sh[t] + ysh[t] * np.float32(sig[t])
    tot_sh = torch.from_numpy(part_sh)
    dist.all_reduce(tot_sh)
    err_sh = float(np.abs(tot_sh.numpy() - full_sh).max() / np.sqrt(np.mean(full_sh.astype(np.float64) ** 2)))
    ranges = [None] * world
    dist.all_gather_object(ranges, (lo, hi))
    if rank == 0:
        ret["err"] = err
        ret["err_shared_dealt"] = err_sh
        ret["ranges"] = ranges
    dist.destroy_process_group()


def test_two_rank_partial_sums_reproduce_the_layer():
    ctx = mp.get_context("spawn")
    with ctx.Manager() as m:
        ret = m.dict()
        procs = [ctx.Process(target=_worker, args=(r, 2, 29517, ret)) for r in range(2)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(120)
            assert p.exitcode == 0
        assert ret["err"] < 1e-6
        assert ret["err_shared_dealt"] < 1e-6
        assert ret["ranges"] == [(0, 5), (5, 10)]


def test_expert_ranges_partition_every_count():
    from flashrt_b200.ep import expert_range
    for E in (512, 10, 7):
        for world in (1, 2, 4, 8):
            r = [expert_range(k, world, E) for k in range(world)]
            assert r[0][0] == 0 and r[-1][1] == E
            assert all(r[i][1] == r[i + 1][0] for i in range(world - 1))


def test_shared_expert_token_ranges_partition_the_tokens_in_whole_items():
    # with the shared expert dealt among the ranks, every token is taken by exactly one rank and the
    # cuts fall on work-item boundaries (four tokens)
    from flashrt_b200.ep import shared_token_range
    for T in (64, 63, 5, 3, 1):
        for world in (1, 2, 4, 8):
            r = [shared_token_range(k, world, T) for k in range(world)]
            assert r[0][0] == 0 and r[-1][1] == T
            assert all(r[i][1] == r[i + 1][0] for i in range(world - 1))
            assert all(lo % 4 == 0 and (hi % 4 == 0 or hi == T) for lo, hi in r)
