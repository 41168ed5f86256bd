"""Expert-parallel layers on two and four real GPUs (one process per GPU, NCCL): the decode form
(replicated tokens, all-reduce) and the prefill form (sharded tokens, all-to-all) against the
single-GPU result. Skipped on machines with fewer GPUs than ranks."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu


def _worker(rank, world, port_no, ret):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port_no), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from flashrt_b200 import ep, moe, synth
    from helpers import Experts, cuda, rel_max
    from oracle import oracle
    port = oracle.port()
    n, ff, E, K, T = 512, 256, 16, 4, 64
    ex = Experts(port, n, ff, E)                       # every rank builds all experts, uses its own range
    lo, hi = ep.expert_range(rank, world, E)
    x, lg = synth.activations(T, n), synth.router_logits(T, E)
    ids, wts, _ = port.route(lg, K)
    # decode form
    out = torch.empty(T, n, device="cuda")
    ids_o = torch.empty(T, K, dtype=torch.int32, device="cuda")
    wts_o = torch.empty(T, K, device="cuda")
    ws = moe.workspace(moe.moe_layer_workspace_bytes(T, K, n, ff))
    ep.moe_layer_ep(ex.base + lo * ex.stride, ex.stride, E, lo, hi, ex.shared_ptr if rank == 0 else None, n, ff, cuda(x), cuda(lg), None, K,
                    out, ids_o, wts_o, ws)
    full = moe.moe_decode(ex.base, ex.stride, E, ex.shared_ptr, n, ff, cuda(x), cuda(ids), cuda(wts), None)
    err_decode = rel_max(out.cpu().numpy(), full.cpu().numpy())
    # decode form with the all-reduce fused into the combine over peer memory: three calls in a row
    # (both buffer slots and a reuse), every rank must end with the same bits
    comm = ep.EpComm(T, n)
    err_fused, same_bits = 0.0, True
    for it in range(3):
        xi = synth.activations(T, n, seed=50 + it)
        want = moe.moe_decode(ex.base, ex.stride, E, ex.shared_ptr, n, ff, cuda(xi), cuda(ids), cuda(wts), None)
        got = torch.empty(T, n, device="cuda")
        if it == 1:   # the shared expert's tokens dealt among the ranks (every rank holds a copy of it)
            ep.moe_layer_ep_fused(comm, ex.base + lo * ex.stride, ex.stride, E, lo, hi, ex.shared_ptr, n, ff, cuda(xi), cuda(lg), None, K, got,
                                  ids_o, wts_o, ws, shared_tokens=ep.shared_token_range(rank, world, T))
        else:         # all of them on rank 0
            ep.moe_layer_ep_fused(comm, ex.base + lo * ex.stride, ex.stride, E, lo, hi, ex.shared_ptr if rank == 0 else None, n, ff, cuda(xi),
                                  cuda(lg), None, K, got, ids_o, wts_o, ws)
        torch.cuda.synchronize()
        moe.workspace_status(ws)
        err_fused = max(err_fused, rel_max(got.cpu().numpy(), want.cpu().numpy()))
        gathered = [torch.empty_like(got) for _ in range(world)]
        dist.all_gather(gathered, got)
        same_bits = same_bits and all(torch.equal(g, gathered[0]) for g in gathered)
    comm.close()
    # prefill form: this rank's half of the tokens
    Tl = T // world
    xs, ls = x[rank * Tl:(rank + 1) * Tl], lg[rank * Tl:(rank + 1) * Tl]
    pipe = ep.PrefillEp(ex.base + lo * ex.stride, ex.stride, E, n, ff, Tl, K, chunks=2)
    o2, i2, w2 = pipe.run(cuda(xs), cuda(ls))
    torch.cuda.synchronize()
    pipe.status()
    ref = port.moe_layer(ex.routed_planar(), ex.blob_bytes, None, n, ff, xs, ids[rank * Tl:(rank + 1) * Tl], wts[rank * Tl:(rank + 1) * Tl])
    err_prefill = rel_max(o2.cpu().numpy(), ref)
    ids_ok = bool(np.array_equal(i2.cpu().numpy(), ids[rank * Tl:(rank + 1) * Tl]))
    ret[rank] = (err_decode, err_prefill, ids_ok, err_fused, same_bits)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_expert_parallel_layers(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    ctx = mp.get_context("spawn")
    with ctx.Manager() as m:
        ret = m.dict()
        procs = [ctx.Process(target=_worker, args=(r, world, 29531 + world, ret)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(180)
            if p.is_alive():
                p.kill()
                pytest.fail("a rank did not finish in time")
            assert p.exitcode == 0
        for r in range(world):
            err_decode, err_prefill, ids_ok, err_fused, same_bits = ret[r]
            assert ids_ok
            assert err_decode < 1e-5 and err_prefill < 1e-5
            assert err_fused < 1e-5 and same_bits
