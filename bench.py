#!/usr/bin/env python
"""Benchmark of the Q2_0 MoE layer: tokens/s through one MoE layer and achieved HBM bandwidth.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--batch B] [--impl reference]

Workload (BASELINE.json configs[1]): one MoE layer decode, hidden 2048, 512 experts of
intermediate 512 plus one shared expert, all Q2_0; router logits fp32 N(0,1), softmax top-10;
batch B tokens (default 64; --batch 1/4/16 give the other decode batches). A *step* is one pass
of B tokens through 48 layers with distinct weights, activations and logits (21.8 GB of experts,
far more than L2, so every layer's weights come from HBM). The value is layer-tokens per second:
B * 48 / step time.

The JSON line carries: `value` with inputs resident in HBM (the 48 layer calls replayed from one
CUDA graph); `e2e` through frx_moe_layers_host with pinned host buffers, copies inside the timed
region; `roofline` of the gate/up streaming kernel from CUDA events around each of its launches;
`cpu_baseline`, the reference's own CPU path (oracle/_ref, AVX-512 moe_cpu on all physical cores)
on a bounded sample of the same workload.

With --gpus N > 1 (launched by torch.distributed.run, one rank per GPU) the experts of every layer
are sharded over the ranks (expert parallel), activations and routing are replicated, and each
layer ends in an all-reduce of the [B][2048] partial sums; total work is fixed ("strong").

--impl reference times the reference's CPU implementation alone, on rank 0.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

N_MODEL, FF, E, K, LAYERS = 2048, 512, 512, 10, 48
EXPERT_BYTES = 884736
GU_BYTES = 589824          # gate + up of one expert
NCU_GU_TRAFFIC_PER_BLOB = 224.33e6 / 367   # DRAM bytes per distinct expert blob of one gate/up launch (ncu, profiles/)
FALLBACK_HBM_GBS = 6650.0
METRIC = "q2_0_moe_layer_tokens_per_s"
UNIT = "layer-tokens/s"


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return float(json.load(open(p))["hbm_gbs"]), "measured (MEASURED_PEAKS.json)"
    return FALLBACK_HBM_GBS, "fallback (6.65 TB/s)"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons, sampled every 50 ms from before the warm-up on; the
    samples that fall inside the timed region (between begin() and stop()) are reported, or, when the
    region was shorter than the sampling period allows, the ones nearest to it (taken under the same
    load, during warm-up)."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.rows, self.proc, self.t_begin = [], None, None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.th = threading.Thread(target=self._read, daemon=True)
            self.th.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [c.strip() for c in line.split(",")]))

    def begin(self):
        self.t_begin = time.time()

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        t_end = time.time()
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        ok = [(t, r) for t, r in self.rows if len(r) >= 6 and r[0].replace(".", "").isdigit()]
        t0 = self.t_begin if self.t_begin is not None else 0.0
        inside = [r for t, r in ok if t0 <= t <= t_end + 0.05]
        window = "timed region"
        if not inside and ok:
            inside = [r for _, r in sorted(ok, key=lambda tr: min(abs(tr[0] - t0), abs(tr[0] - t_end)))[:3]]
            window = "nearest samples (region shorter than the sampling period)"
        sm = [float(r[0]) for r in inside]
        mx = [float(r[1]) for r in inside if r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].lower() == "active" for r in inside)]
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(sm), "window": window}


def cpu_moe_setup(oracle, n_layers: int, B: int, seed: int):
    """Host-side planar experts (E routed + the shared expert as expert E), activations and routing
    for the CPU legs."""
    from flashrt_b200 import synth
    port = oracle.port()
    rng = np.random.default_rng(seed)
    planar = synth.planar_experts_random(rng, n_layers * (E + 1), N_MODEL, FF).reshape(n_layers, E + 1, EXPERT_BYTES)
    x = rng.standard_normal((n_layers, B, N_MODEL), dtype=np.float32)
    ids = np.empty((n_layers, B, K + 1), np.int32)
    wts = np.empty((n_layers, B, K + 1), np.float32)
    for l in range(n_layers):
        i, w, _ = port.route(rng.standard_normal((B, E), dtype=np.float32), K)
        gate = rng.standard_normal(B).astype(np.float32)
        ids[l, :, :K], wts[l, :, :K] = i, w
        ids[l, :, K] = E                                         # the shared expert: one more entry,
        wts[l, :, K] = 1.0 / (1.0 + np.exp(-gate))               # weighted by sigmoid(gate)
    return planar, x, ids, wts


def time_cpu(ref, planar, x, ids, wts, workers: int, reps: int) -> float:
    n_layers, B = x.shape[0], x.shape[1]
    return ref.moe_cpu_timed(planar, EXPERT_BYTES, (E + 1) * EXPERT_BYTES, n_layers, E + 1, N_MODEL, FF, x, ids, wts, workers, reps)


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import oracle
    ref = oracle.ref()
    B = args.batch
    if ref is None:
        print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref/libfrx_ref.so was not built (needs the reference tree)"}))
        return
    cpu_layers = 3
    planar, x, ids, wts = cpu_moe_setup(oracle, cpu_layers, B, seed=20260927)
    workers = max(1, ref.physical_cpus())
    for _ in range(args.warmup):
        time_cpu(ref, planar, x, ids, wts, workers, cpu_layers)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        time_cpu(ref, planar, x, ids, wts, workers, cpu_layers)
    dt = time.perf_counter() - t0
    ms = dt / args.steps * 1e3
    value = B * cpu_layers / (dt / args.steps)
    sample = f"{cpu_layers} layers x {B} tokens per step (1.36 GB of experts), quantize + entry lists + moe_cpu per layer"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "int8 x 2-bit dot, fp32 scale/accumulate", "data": "synthetic",
        "config": {"workload": f"configs[1]: one Q2_0 MoE layer decode, batch {B}, hidden 2048, 512 experts + shared, top-10",
                   "batch": B, "layers_per_step": cpu_layers},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": workers, "kind": "reference", "sample": sample,
                         "avx512_vnni": ref.have_avx512()},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def run_frx(args):
    import torch
    import torch.distributed as dist

    from flashrt_b200 import moe

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    B, L = args.batch, args.layers
    if args.nw:
        moe.check(moe.lib.frx_debug_set_consumer_warps(args.nw))
    if args.narrow is not None:
        moe.check(moe.lib.frx_debug_set_narrow_items(args.narrow))
    e_lo, e_hi = rank * E // world, (rank + 1) * E // world
    e_local = e_hi - e_lo

    # ---- weights: per layer, this rank's experts plus the shared expert, generated on the device
    arena = moe.ExpertArena(L, e_local + 1, N_MODEL, FF)
    gen = torch.Generator(device=dev)
    nb_gu, nb_dn = FF * (N_MODEL // 64), N_MODEL * (FF // 64)

    def layer_planar(l: int) -> torch.Tensor:
        """Layer l's E + 1 planar blobs (the same bytes on every rank): uniform codes, scales |N(0, 0.02)|."""
        gen.manual_seed(20260927 + l)
        p = torch.randint(0, 256, (E + 1, EXPERT_BYTES), dtype=torch.uint8, device=dev, generator=gen)
        off = 0
        for nblk in (nb_gu, nb_gu, nb_dn):
            d = (torch.randn(E + 1, nblk, device=dev, generator=gen) * 0.02).abs().to(torch.float16)
            d[d == 0] = 6.103515625e-05
            p[:, off + nblk * 16:off + nblk * 18] = d.view(torch.uint8).view(E + 1, nblk * 2)
            off += nblk * 18
        return p

    keep = {}
    for l in range(L):
        p = layer_planar(l)
        mine = torch.cat([p[e_lo:e_hi], p[E:E + 1]]).contiguous()
        arena.load_planar(l, 0, e_local + 1, mine.view(-1))
        if l < 2 and rank == 0:
            keep[l] = p.cpu().numpy()
        del p, mine
    torch.cuda.synchronize()

    gen.manual_seed(7)
    x = torch.randn(L, B, N_MODEL, device=dev, generator=gen)
    gen.manual_seed(9)
    logits = torch.randn(L, B, E, device=dev, generator=gen)
    gate = torch.randn(L, B, device=dev, generator=gen)
    out = torch.empty(L, B, N_MODEL, device=dev)
    ids = torch.empty(L, B, K, dtype=torch.int32, device=dev)
    wts = torch.empty(L, B, K, device=dev)
    ws = moe.workspace(moe.moe_layer_workspace_bytes(B, K, N_MODEL, FF), dev)

    # Expert parallel: the all-reduce is fused into each layer's last kernel over peer memory (CUDA
    # IPC); if the peer mapping cannot be set up, NCCL's all-reduce is used instead.
    comm = None
    if world > 1:
        from flashrt_b200 import ep
        try:
            comm = ep.EpComm(B, N_MODEL)
        except Exception as exc:   # noqa: BLE001 - any failure of the set-up means the NCCL form
            if rank == 0:
                print(f"peer-memory all-reduce unavailable ({exc}); using NCCL", file=sys.stderr)
        ok = torch.tensor([1 if comm is not None else 0], device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if int(ok.item()) == 0:   # some rank could not map its peers: every rank takes part in the ordered tear-down
            torch.cuda.synchronize()
            dist.barrier()
            if comm is not None:
                comm.close_mappings()
            dist.barrier()
            if comm is not None:
                comm.destroy()
            comm = None

    def ep_layer(l: int, xin, lin, gin, o):
        shared_blob = arena.blob(l, e_local) if rank == 0 else None
        if comm is not None:
            ep.moe_layer_ep_fused(comm, arena.blob(l, 0), arena.stride, E, e_lo, e_hi, shared_blob, N_MODEL, FF, xin, lin, gin, K, o,
                                  ids[l], wts[l], ws)
        else:
            ep.moe_layer_ep(arena.blob(l, 0), arena.stride, E, e_lo, e_hi, shared_blob, N_MODEL, FF, xin, lin, gin, K, o, ids[l], wts[l], ws)

    def layer_call(l: int):
        if world == 1:
            moe.moe_layer(arena.blob(l, 0), arena.stride, E, arena.blob(l, e_local), N_MODEL, FF, x[l], logits[l], gate[l], K,
                          out=out[l], ids_out=ids[l], wts_out=wts[l], ws=ws)
        else:
            ep_layer(l, x[l], logits[l], gate[l], out[l])

    def step():
        for l in range(L):
            layer_call(l)

    if world > 1:   # the ranks' set-up times differ; the fused all-reduce waits for a peer for 2 s at most
        torch.cuda.synchronize()
        dist.barrier()
    step()
    if comm is not None:
        # the fused all-reduce reports a peer that did not answer in time through the workspace status;
        # if any rank saw that, every rank drops to the NCCL form (with a fresh workspace: the status sticks)
        try:
            moe.workspace_status(ws)
            fused_ok = 1
        except moe.FrxError as exc:
            fused_ok = 0
            print(f"rank {rank}: fused all-reduce failed ({exc}); using NCCL", file=sys.stderr)
        flag = torch.tensor([fused_ok], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if int(flag.item()) == 0:
            comm.close()
            comm = None
            ws = moe.workspace(moe.moe_layer_workspace_bytes(B, K, N_MODEL, FF), dev)
            step()
    moe.workspace_status(ws)
    torch.cuda.synchronize()
    distinct = [int(torch.unique(ids[l]).numel()) for l in range(L)]
    local_distinct = [int(((torch.unique(ids[l]) >= e_lo) & (torch.unique(ids[l]) < e_hi)).sum()) for l in range(L)]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- value: inputs resident in HBM; the 48 layer calls replayed from one CUDA graph. With
    # NCCL all-reduces on the path the launches stay plain (capturing them together with these
    # kernels did not complete on the 2-GPU box, so it is not attempted).
    use_graph = (world == 1 or comm is not None) and not args.no_graph
    run = step
    if use_graph:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            step()
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            step()
        run = graph.replay
    sampler = ClockSampler(local) if rank == 0 else None
    for _ in range(args.warmup):
        run()
    barrier()
    if sampler:
        sampler.begin()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        run()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1) / args.steps
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    moe.workspace_status(ws)
    value = B * L / (ms * 1e-3)

    # ---- per-kernel device time: CUDA events around every launch, the same K steps without the graph
    ncls = 8
    pms, pn = (C.c_float * ncls)(), (C.c_int * ncls)()
    moe.check(moe.lib.frx_profile_begin())
    for _ in range(args.steps):
        step()
    moe.check(moe.lib.frx_profile_end(pms, pn, ncls))
    clocks = sampler.stop() if sampler else None
    names = [moe.lib.frx_profile_class_name(i).decode() for i in range(ncls)]
    kernels = {names[i]: {"launches": int(pn[i]), "ms_total": round(float(pms[i]), 4),
                          "us_per_launch": round(1e3 * float(pms[i]) / max(1, int(pn[i])), 3)} for i in range(ncls) if pn[i]}
    gu_us = kernels["gate_up"]["us_per_launch"]
    peak, peak_src = peaks()
    mean_local = float(np.mean(local_distinct)) + (1.0 if rank == 0 or world == 1 else 0.0)
    gu_alg_bytes = mean_local * GU_BYTES + B * (N_MODEL + N_MODEL // 32 * 8) + B * (K + 1) * FF * 4
    achieved = gu_alg_bytes / (gu_us * 1e-6) / 1e9
    layer_bytes = float(np.mean([(d + 1) * EXPERT_BYTES for d in distinct])) + B * (E * 4 + N_MODEL * 8) + B * K * 8
    roofline = {"bound": "hbm", "kernel": "k_stream<gate_up>", "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
                "frac": round(achieved / peak, 4), "peak_source": peak_src,
                # dram__bytes_read.sum + dram__bytes_write.sum of one launch: 224.33 MB for 367 distinct
                # expert blobs in the ncu capture summarised in profiles/k_stream_decode_b64.md (a 2-layer
                # case of the same kernel), scaled to this run by the distinct blobs a launch reads
                "traffic": int(mean_local * NCU_GU_TRAFFIC_PER_BLOB), "traffic_source": "ncu capture of a 2-layer case, scaled by distinct expert blobs",
                "algorithmic_bytes_per_launch": int(gu_alg_bytes), "us_per_launch": gu_us,
                "timing": "CUDA events around each launch, a separate pass of the same steps without the CUDA graph",
                "layer": {"algorithmic_bytes": int(layer_bytes), "us": round(ms * 1e3 / L, 3),
                          "achieved_GBps": round(layer_bytes / world / (ms * 1e-3 / L) / 1e9, 1),
                          "frac_of_peak": round(layer_bytes / world / (ms * 1e-3 / L) / 1e9 / peak, 4)}}

    # ---- e2e: host buffers through frx_moe_layers_host (one call per step, copies pipelined with
    # compute), every copy inside the timed region
    e2e = None
    if world == 1:
        xh, lh, gh = x.cpu().pin_memory(), logits.cpu().pin_memory(), gate.cpu().pin_memory()
        oh = torch.empty(L, B, N_MODEL).pin_memory()
        hws = moe.workspace(moe.moe_layers_host_workspace_bytes(B, K, N_MODEL, FF, E), dev)
        blobs, shared_blobs = [arena.blob(l, 0) for l in range(L)], [arena.blob(l, e_local) for l in range(L)]
        xl, ll, gl, ol = [xh[l] for l in range(L)], [lh[l] for l in range(L)], [gh[l] for l in range(L)], [oh[l] for l in range(L)]

        def host_step():   # one call: the step's 48 layers from pinned host buffers, results back in host memory
            moe.moe_layers_host(blobs, arena.stride, E, shared_blobs, N_MODEL, FF, xl, ll, gl, K, ol, hws)

        for _ in range(max(1, args.warmup // 2)):
            host_step()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            host_step()
        torch.cuda.synchronize()
        e2e_ms = (time.perf_counter() - t0) / args.steps * 1e3
        assert torch.equal(oh.to(dev), out), "host entry and device entry disagree"
        e2e = {"value": B * L / (e2e_ms * 1e-3), "unit": UNIT, "ms_per_step": round(e2e_ms, 4),
               "h2d_bytes_per_step": L * B * (N_MODEL + E + 1) * 4, "d2h_bytes_per_step": L * B * N_MODEL * 4}
    else:
        # Expert parallel: the activations and logits are replicated, so every rank copies its own
        # from pinned host memory; the all-reduced result goes back to host memory on every rank.
        # Copies, layer calls and all-reduces are stream-ordered; one synchronisation per step.
        xh, lh, gh = x.cpu().pin_memory(), logits.cpu().pin_memory(), gate.cpu().pin_memory()
        oh = torch.empty(L, B, N_MODEL).pin_memory()
        # two staging sets and two copy streams, so that a layer's compute overlaps the copy-in of the
        # next layer and the copy-out of the previous one (what frx_moe_layers_host does on one GPU)
        NB = 2
        xd = [torch.empty_like(x[0]) for _ in range(NB)]
        ld = [torch.empty_like(logits[0]) for _ in range(NB)]
        gd = [torch.empty_like(gate[0]) for _ in range(NB)]
        od = [torch.empty_like(out[0]) for _ in range(NB)]
        s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
        ev_in = [torch.cuda.Event() for _ in range(NB)]
        ev_done = [torch.cuda.Event() for _ in range(NB)]
        ev_out = [torch.cuda.Event() for _ in range(NB)]

        def host_step():
            main = torch.cuda.current_stream()
            s_in.wait_stream(main)
            for l in range(L):
                b = l % NB
                with torch.cuda.stream(s_in):
                    if l >= NB:
                        s_in.wait_event(ev_done[b])   # the layer that read this staging set has run
                    xd[b].copy_(xh[l], non_blocking=True)
                    ld[b].copy_(lh[l], non_blocking=True)
                    gd[b].copy_(gh[l], non_blocking=True)
                    ev_in[b].record(s_in)
                main.wait_event(ev_in[b])
                if l >= NB:
                    main.wait_event(ev_out[b])        # its previous output has been copied out
                ep_layer(l, xd[b], ld[b], gd[b], od[b])
                ev_done[b].record(main)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_done[b])
                    oh[l].copy_(od[b], non_blocking=True)
                    ev_out[b].record(s_out)
            torch.cuda.synchronize()

        barrier()
        for _ in range(max(1, args.warmup // 2)):
            host_step()
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            host_step()
        barrier()
        e2e_ms = (time.perf_counter() - t0) / args.steps * 1e3
        t = torch.tensor([e2e_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
        assert torch.allclose(oh.to(dev), out, rtol=1e-5, atol=1e-6), "host-buffer step and device-resident step disagree"
        e2e = {"value": B * L / (e2e_ms * 1e-3), "unit": UNIT, "ms_per_step": round(e2e_ms, 4),
               "h2d_bytes_per_step": world * L * B * (N_MODEL + E + 1) * 4, "d2h_bytes_per_step": world * L * B * N_MODEL * 4}

    # ---- CPU baseline: the reference's CPU path on a bounded sample (rank 0, single GPU runs only)
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        from oracle import oracle
        ref = oracle.ref()
        if ref is not None:
            nl = len(keep)
            planar = np.stack([keep[l] for l in range(nl)])
            idh = np.concatenate([ids[:nl].cpu().numpy(), np.full((nl, B, 1), E, np.int32)], axis=2)
            gsig = torch.sigmoid(gate[:nl]).cpu().numpy()[..., None]
            wth = np.concatenate([wts[:nl].cpu().numpy(), gsig], axis=2).astype(np.float32)
            workers = max(1, ref.physical_cpus())
            xs = x[:nl].cpu().numpy()
            t1 = time_cpu(ref, planar, xs, idh, wth, workers, nl)
            reps = int(min(400, max(2 * nl, 12.0 / max(t1, 1e-6))))
            sec = time_cpu(ref, planar, xs, idh, wth, workers, reps)
            cpu = {"value": B / sec, "unit": UNIT, "cores": workers, "kind": "reference",
                   "sample": f"{reps} moe_cpu layer calls over {nl} layers x {B} tokens (same weights, routing and activations "
                             f"as the GPU run), {sec * 1e3:.3f} ms per layer", "avx512_vnni": ref.have_avx512()}
            # the GPU result against the reference's CPU result on the same inputs
            o = ref.moe_cpu(planar[0], EXPERT_BYTES, E + 1, N_MODEL, FF, xs[0], idh[0], wth[0], workers=workers)
            got = out[0].cpu().numpy()
            cpu["gpu_vs_cpu_max_err_over_rms"] = float(np.abs(got - o).max() / np.sqrt(np.mean(o.astype(np.float64) ** 2)))
        else:
            cpu = {"value": None, "unit": UNIT, "cores": 0, "kind": "reference", "sample": "oracle/_ref not built"}

    if world > 1:   # every rank must hold the same routing and the same reduced output
        chk = torch.stack([out.double().sum(), ids.double().sum()])
        lo_, hi_ = chk.clone(), chk.clone()
        dist.all_reduce(lo_, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi_, op=dist.ReduceOp.MAX)
        assert torch.equal(lo_, hi_), "ranks disagree on the layer output"
    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "int8 x 2-bit dot, fp32 scale/accumulate", "data": "synthetic",
            "config": {"workload": f"configs[1]: one Q2_0 MoE layer decode, batch {B}, hidden 2048, 512 experts + shared, top-10",
                       "batch": B, "layers_per_step": L, "l2": "inputs larger than L2: 48 distinct layers, 21.8 GB of experts",
                       "distinct_experts_per_layer_mean": float(np.mean(distinct)), "parallelism": f"ep{world}",
                       "cuda_graph": use_graph,
                       "all_reduce": "none" if world == 1 else ("fused into the combine kernel, peer memory over NVLink" if comm is not None else "NCCL")},
            "clocks": clocks, "e2e": e2e, "gpu_launches": sum(v["launches"] for v in kernels.values()), "kernels": kernels,
            "roofline": roofline, "cpu_baseline": cpu,
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def run_prefill(args):
    """BASELINE.json configs[2] (one GPU) and configs[4] (expert parallel, --gpus N under
    torch.distributed.run): one MoE layer prefill of --tokens tokens x hidden 2048 (bf16-rounded
    N(0,1)), 512 experts top-10, Zipf(1.1) or uniform routing. A step is route + grouped expert
    product + combine; expert parallel, tokens and experts are both sharded over the ranks and the
    slots travel by NCCL all-to-all."""
    import torch
    import torch.distributed as dist

    from flashrt_b200 import ep, moe, synth

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    T = args.tokens
    Tl = T // world
    e_lo, e_hi = ep.expert_range(rank, world, E)
    arena = moe.ExpertArena(1, e_hi - e_lo, N_MODEL, FF)
    gen = torch.Generator(device=dev)
    gen.manual_seed(20260927)
    nb_gu, nb_dn = FF * (N_MODEL // 64), N_MODEL * (FF // 64)
    pl = torch.randint(0, 256, (E, EXPERT_BYTES), dtype=torch.uint8, device=dev, generator=gen)
    off = 0
    for nblk in (nb_gu, nb_gu, nb_dn):
        d = (torch.randn(E, nblk, device=dev, generator=gen) * 0.02).abs().to(torch.float16)
        d[d == 0] = 6.103515625e-05
        pl[:, off + nblk * 16:off + nblk * 18] = d.view(torch.uint8).view(E, nblk * 2)
        off += nblk * 18
    arena.load_planar(0, 0, e_hi - e_lo, pl[e_lo:e_hi].contiguous().view(-1))
    del pl
    xa = synth.activations(T, N_MODEL, through_bf16=True)
    la = synth.zipf_logits(T, E) if args.routing == "zipf" else synth.router_logits(T, E)
    x = torch.from_numpy(xa[rank * Tl:(rank + 1) * Tl]).to(dev)
    logits = torch.from_numpy(la[rank * Tl:(rank + 1) * Tl]).to(dev)
    ws = moe.workspace(moe.moe_q2.workspace_bytes(Tl, K, N_MODEL, FF, E), dev)
    yd = torch.empty(Tl * K, N_MODEL, device=dev)
    out = torch.empty(Tl, N_MODEL, device=dev)

    def step():
        if world == 1:
            ids, wts = moe.moe_route_topk(logits, K)
            moe.moe_q2.run(arena.blob(0, 0), arena.stride, E, N_MODEL, FF, x, ids, yd=yd, ws=ws, form=args.form)
            moe.moe_combine(yd.view(Tl, K, N_MODEL), wts, None, None, None, out=out)
        else:
            ep.moe_prefill_ep(arena.blob(0, 0), arena.stride, E, N_MODEL, FF, x, logits, K)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local) if rank == 0 else None
    for _ in range(args.warmup):
        step()
    moe.workspace_status(ws)
    barrier()
    if sampler:
        sampler.begin()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1) / args.steps
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ncls = 8
    pms, pn = (C.c_float * ncls)(), (C.c_int * ncls)()
    moe.check(moe.lib.frx_profile_begin())
    for _ in range(args.steps):
        step()
    moe.check(moe.lib.frx_profile_end(pms, pn, ncls))
    clocks = sampler.stop() if sampler else None
    names = [moe.lib.frx_profile_class_name(i).decode() for i in range(ncls)]
    kernels = {names[i]: {"launches": int(pn[i]), "us_per_step": round(1e3 * float(pms[i]) / args.steps, 2)} for i in range(ncls) if pn[i]}
    flops = T * K * 3 * 2 * N_MODEL * FF
    gu_ms, dn_ms = kernels["gate_up"]["us_per_step"] / 1e3, kernels["down"]["us_per_step"] / 1e3
    peak_tf = 1657.0
    pk = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(pk):
        peak_tf = float(json.load(open(pk))["bf16_tflops"])
    gemm_tf = flops / world / ((gu_ms + dn_ms) * 1e-3) / 1e12
    if rank == 0:
        print(json.dumps({
            "metric": "q2_0_moe_prefill_tokens_per_s", "value": T / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "dtype": "exact integer products (int8 / fp16 operands), fp32 scale and accumulate", "data": "synthetic",
            "config": {"workload": f"configs[{2 if world == 1 else 4}]: one Q2_0 MoE layer prefill, {T} tokens, hidden 2048, 512 experts top-10, "
                                   f"{'Zipf(1.1)' if args.routing == 'zipf' else 'uniform'} routing",
                       "form": args.form, "parallelism": f"ep{world}", "l2": "453 MB of experts per step, larger than L2"},
            "clocks": clocks, "kernels": kernels,
            "roofline": {"bound": "tensor", "kernel": "expert product (gate/up + down), rank 0", "achieved": round(gemm_tf, 1), "peak": peak_tf,
                         "unit": "TFLOP/s", "frac": round(gemm_tf / peak_tf, 4), "flops_per_step": flops, "ms_gate_up": gu_ms,
                         "ms_down": dn_ms, "traffic": None}}))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="frx", choices=["frx", "reference"])
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--layers", type=int, default=LAYERS)
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--nw", type=int, default=0, help="tuning: consumer warps of the streaming kernel (8, 12, 16)")
    ap.add_argument("--narrow", type=int, default=None, help="tuning: 0 sends every work item through the eight-token form")
    ap.add_argument("--workload", default="decode", choices=["decode", "prefill"], help="decode = configs[1] (default), prefill = configs[2]")
    ap.add_argument("--tokens", type=int, default=4096, help="prefill tokens")
    ap.add_argument("--routing", default="zipf", choices=["zipf", "uniform"], help="prefill routing skew")
    ap.add_argument("--form", default="auto", choices=["auto", "umma", "stream"], help="prefill kernel form")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "prefill":
        run_prefill(args)
    else:
        run_frx(args)


if __name__ == "__main__":
    main()
