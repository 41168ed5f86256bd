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
on a bounded sample of the same workload. The headline keys describe configs[1] at batch 64; the
other configurations ride along in the same line, each with its own parity figure against the
CPU oracle at the full shape (512 experts):
  `decode_batches`  configs[1] at batch 1, 4 and 16: us per layer, layer-tokens/s, fraction of the HBM peak;
  `prefill`         configs[2] (one GPU: 4,096 tokens, Zipf routing) or configs[4] (--gpus N: 16,384
                    tokens, uniform and Zipf routing, expert parallel): tokens/s, TFLOP/s of the
                    expert products, fraction of the measured bf16 peak, the kernel form taken;
  `verify_stack`    configs[3]: the 48 layers chained (x_next = rmsnorm_unit(x + y)) for a window of
                    three tokens: tokens/s, us per layer, HBM fraction (latency-limited by nature).

With --gpus N > 1 (launched by torch.distributed.run, one rank per GPU) the experts of every layer
are sharded over the ranks (expert parallel), activations and routing are replicated, the shared
expert's tokens are dealt among the ranks, and each layer ends in an all-reduce of the [B][2048]
partial sums inside its last kernel; total work is fixed ("strong"). The line then also carries
`ep_allreduce`: where that kernel's time goes on every rank (its own cycle stamps).

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
NCU_FFN_TRAFFIC_PER_BLOB = None            # the same for one launch of the fused kernel (k_ffn)
NCU_GU_TRAFFIC_PER_BLOB = 223.7e6 / 367    # DRAM read + write bytes per distinct expert blob of one gate/up launch (an ncu capture of a 2-layer case)
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


def cpu_workers_sweep(ref, planar, x, ids, wts, reps: int = 24) -> dict:
    """The reference's moe_cpu at its own sweet spots (6 and 8 workers) and on all physical cores:
    mean, median and 99th percentile of the time of one layer call, and the implied weight bandwidth."""
    n_layers, B = x.shape[0], x.shape[1]
    allc = max(1, ref.physical_cpus())
    out = {}
    for w in sorted({min(6, allc), min(8, allc), allc}):
        secs = ref.moe_cpu_times(planar, EXPERT_BYTES, (E + 1) * EXPERT_BYTES, n_layers, E + 1, N_MODEL, FF, x, ids, wts, w, reps)[n_layers:]
        distinct = float(np.mean([len(np.unique(ids[l])) for l in range(n_layers)]))
        out[str(w)] = {"mean_us": round(float(secs.mean()) * 1e6, 1), "p50_us": round(float(np.percentile(secs, 50)) * 1e6, 1),
                       "p99_us": round(float(np.percentile(secs, 99)) * 1e6, 1), "calls": int(secs.size),
                       "weight_GBps": round(distinct * EXPERT_BYTES / float(secs.mean()) / 1e9, 1)}
    return out


def cpu_config0(ref) -> dict:
    """BASELINE configs[0]: one Q2_0 expert GEMV (512 x 2048, batch 1) on one host thread, the
    reference's AVX-512 kernel and its scalar form, with the matrix in cache and streamed from DRAM
    (a ring of 1,024 matrices, 300 MB)."""
    from flashrt_b200 import synth
    rng = np.random.default_rng(synth.SEED_WEIGHTS)
    rows, cols, mb = 512, 2048, 294912
    ring = 1024
    mats = rng.integers(0, 256, size=ring * mb, dtype=np.uint8)
    d = np.abs(rng.standard_normal(ring * rows * (cols // 64), dtype=np.float32) * np.float32(0.02)).astype(np.float16)
    d[d == 0] = np.float16(6.103515625e-05)
    mats.reshape(ring, mb)[:, rows * (cols // 64) * 16:] = d.view(np.uint8).reshape(ring, -1)
    x = synth.activations(1, cols)[0]
    alg = mb + cols + cols // 32 * 4 + rows * 4          # weights + Q8 activation + output
    res = {"shape": "512 x 2048 (out x in), batch 1, one thread", "algorithmic_bytes": alg}
    for name, avx, reps_c, reps_d in (("matvec_avx512", True, 4000, 4096), ("matvec_ref", False, 60, 64)):
        if avx and not ref.have_avx512():
            continue
        sec_c, y_c = ref.matvec_timed(mats, 1, rows, cols, x, avx, reps_c)
        sec_d, _ = ref.matvec_timed(mats, ring, rows, cols, x, avx, reps_d)
        res[name] = {"cached_us": round(sec_c * 1e6, 2), "dram_us": round(sec_d * 1e6, 2), "dram_GBps": round(alg / sec_d / 1e9, 2)}
        res.setdefault("_y", {})[name] = y_c
    if "matvec_avx512" in res.get("_y", {}) and "matvec_ref" in res["_y"]:
        a, b = res["_y"]["matvec_avx512"], res["_y"]["matvec_ref"]
        res["avx512_vs_scalar_max_err_over_rms"] = float(np.abs(a - b).max() / np.sqrt(np.mean(b.astype(np.float64) ** 2)))
    res.pop("_y", None)
    return res


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
    sweep = cpu_workers_sweep(ref, planar, x, ids, wts)
    config0 = cpu_config0(ref)
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "int8 x 2-bit dot, fp32 scale/accumulate", "data": "synthetic",
        "config": {"workload": f"configs[1]: one Q2_0 MoE layer decode, batch {B}, hidden 2048, 512 experts + shared, top-10",
                   "batch": B, "layers_per_step": cpu_layers},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": workers, "kind": "reference", "sample": sample,
                         "avx512_vnni": ref.have_avx512(), "workers_sweep": sweep},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "config0": config0,
    }))


def rel_max(a, b) -> float:
    """max |a - b| over the RMS of b (the reference's error measure, tests/test_q2_0.cpp:117-124)."""
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.abs(a - b).max() / max(np.sqrt(np.mean(b ** 2)), 1e-30))


def run_frx(args):
    import torch
    import torch.distributed as dist

    from flashrt_b200 import moe, synth

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
    if args.fused is not None:
        moe.check(moe.lib.frx_debug_set_fused_ffn(args.fused))
    if args.down_weight is not None:
        moe.check(moe.lib.frx_debug_set_down_task_weight(args.down_weight))
    if args.evict_first is not None:
        moe.check(moe.lib.frx_debug_set_evict_first(args.evict_first))
    if args.down_item_weight is not None:
        moe.check(moe.lib.frx_debug_set_down_item_weight(args.down_item_weight))
    if args.small_limits:
        moe.check(moe.lib.frx_debug_set_small_launch_limits(*[int(v) for v in args.small_limits.split(",")]))
    if args.fold is not None:
        moe.check(moe.lib.frx_debug_set_fold_quant(args.fold))
    if args.ffn_buffers:
        moe.check(moe.lib.frx_debug_set_ffn_buffers(*[int(v) for v in args.ffn_buffers.split(",")]))
    if args.task4 is not None:
        moe.check(moe.lib.frx_debug_set_four_group_tasks(args.task4))
    if args.gu_chunks:
        moe.check(moe.lib.frx_debug_set_gate_up_chunks(args.gu_chunks))
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

    def layer(l: int, xin, lin, gin, o, ids_l, wts_l, ws_):
        """One MoE layer call on device tensors: the plain entry on one GPU, the expert-parallel one otherwise."""
        if world == 1:
            moe.moe_layer(arena.blob(l, 0), arena.stride, E, arena.blob(l, e_local), N_MODEL, FF, xin, lin, gin, K,
                          out=o, ids_out=ids_l, wts_out=wts_l, ws=ws_)
            return
        if comm is not None:   # every rank holds the shared expert and applies it to its share of the tokens
            ep.moe_layer_ep_fused(comm, arena.blob(l, 0), arena.stride, E, e_lo, e_hi, arena.blob(l, e_local), N_MODEL, FF, xin, lin, gin, K, o,
                                  ids_l, wts_l, ws_, shared_tokens=ep.shared_token_range(rank, world, xin.shape[0]) if args.deal_shared else
                                  ((0, xin.shape[0]) if rank == 0 else (0, 0)))
            return
        ep.moe_layer_ep(arena.blob(l, 0), arena.stride, E, e_lo, e_hi, arena.blob(l, e_local) if rank == 0 else None, N_MODEL, FF, xin, lin, gin, K,
                        o, ids_l, wts_l, ws_)

    def ep_layer(l: int, xin, lin, gin, o):
        layer(l, xin, lin, gin, o, ids[l], wts[l], ws)

    def step():
        for l in range(L):
            layer(l, x[l], logits[l], gate[l], out[l], ids[l], wts[l], ws)

    if world > 1:   # the ranks' set-up times differ; the fused all-reduce waits for a peer for 2 s at most
        torch.cuda.synchronize()
        dist.barrier()
    step()
    if comm is not None:
        # the fused all-reduce reports a peer that did not answer in time through the workspace status;
        # if any rank saw that, every rank drops to the NCCL form
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
            step()
    moe.workspace_status(ws)
    torch.cuda.synchronize()
    distinct = [int(torch.unique(ids[l]).numel()) for l in range(L)]
    local_distinct = [int(((torch.unique(ids[l]) >= e_lo) & (torch.unique(ids[l]) < e_hi)).sum()) for l in range(L)]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # With NCCL all-reduces on the path the launches stay plain: a capture of NCCL collectives
    # together with these kernels once failed to complete, so it is not attempted.
    use_graph = (world == 1 or comm is not None) and not args.no_graph

    def timeit(fn, warmup: int, steps: int) -> float:
        """Milliseconds per call of fn (device time by CUDA events, the maximum over the ranks); fn is
        replayed from one CUDA graph where that is possible."""
        run = fn
        if use_graph:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                fn()
            torch.cuda.current_stream().wait_stream(side)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                fn()
            run = graph.replay
        for _ in range(warmup):
            run()
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            run()
        b.record()
        barrier()
        t = a.elapsed_time(b) / steps
        if world > 1:
            tt = torch.tensor([t], device=dev)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            t = float(tt.item())
        return t

    # ---- value: inputs resident in HBM; the 48 layer calls replayed from one CUDA graph
    sampler = ClockSampler(local) if rank == 0 else None
    begun = [False]

    def timed_region_begins():
        if sampler and not begun[0]:
            sampler.begin()
            begun[0] = True

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
    for _ in range(args.warmup):
        run()
    barrier()
    timed_region_begins()
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
    ncls = 16
    pms, pn = (C.c_float * ncls)(), (C.c_int * ncls)()
    moe.check(moe.lib.frx_profile_begin())
    for _ in range(args.steps):
        step()
    moe.check(moe.lib.frx_profile_end(pms, pn, ncls))
    clocks = sampler.stop() if sampler else None
    names = [moe.lib.frx_profile_class_name(i).decode() for i in range(ncls)]
    kernels = {names[i]: {"launches": int(pn[i]), "ms_total": round(float(pms[i]), 4),
                          "us_per_launch": round(1e3 * float(pms[i]) / max(1, int(pn[i])), 3)} for i in range(ncls) if pn[i]}
    peak, peak_src = peaks()
    mean_local = float(np.mean(local_distinct)) + (1.0 if rank == 0 or world == 1 else 0.0)
    fused = "ffn" in kernels   # gate/up, the hidden rows and down in one kernel (k_ffn), else k_stream<gate_up> is the dominant kernel
    if fused:
        # whole blobs, the quantized x in, (gate x, up x) pairs out and in again, the slots' output rows out
        top_name, gu_us = "k_ffn", kernels["ffn"]["us_per_launch"]
        gu_alg_bytes = (mean_local * EXPERT_BYTES + B * (N_MODEL + N_MODEL // 32 * 8) + 2 * B * (K + 1) * FF * 8
                        + B * (K + 1) * N_MODEL * 4)
        traffic_per_blob = NCU_FFN_TRAFFIC_PER_BLOB
    else:
        top_name, gu_us = "k_stream<gate_up>", kernels["gate_up"]["us_per_launch"]
        gu_alg_bytes = mean_local * GU_BYTES + B * (N_MODEL + N_MODEL // 32 * 8) + B * (K + 1) * FF * 4
        traffic_per_blob = NCU_GU_TRAFFIC_PER_BLOB
    achieved = gu_alg_bytes / (gu_us * 1e-6) / 1e9

    def layer_alg_bytes(dist_list, Bt):
        return float(np.mean([(d + 1) * EXPERT_BYTES for d in dist_list])) + Bt * (E * 4 + N_MODEL * 8) + Bt * K * 8

    layer_bytes = layer_alg_bytes(distinct, B)
    roofline = {"bound": "hbm", "kernel": top_name, "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
                "frac": round(achieved / peak, 4), "peak_source": peak_src,
                # dram__bytes_read.sum + dram__bytes_write.sum of one launch, from an ncu capture of a 2-layer
                # case of the same kernel, scaled to this run by the distinct blobs a launch reads
                "traffic": int(mean_local * traffic_per_blob) if traffic_per_blob else None, "traffic_source": "ncu capture of a 2-layer case, scaled by distinct expert blobs",
                "algorithmic_bytes_per_launch": int(gu_alg_bytes), "us_per_launch": gu_us,
                "timing": "CUDA events around each launch, a separate pass of the same steps without the CUDA graph",
                "layer": {"algorithmic_bytes": int(layer_bytes), "us": round(ms * 1e3 / L, 3),
                          "achieved_GBps": round(layer_bytes / world / (ms * 1e-3 / L) / 1e9, 1),
                          "frac_of_peak": round(layer_bytes / world / (ms * 1e-3 / L) / 1e9 / peak, 4)}}

    # ---- expert parallel: where the fused all-reduce's time goes (SM cycle stamps of block 0 in the last
    # layer call of the pass above, every rank's)
    ep_allreduce = None
    if comm is not None:
        st = comm.stamps()
        mine = torch.tensor([st[1] - st[0], st[2] - st[1], st[3] - st[2]], dtype=torch.float64, device=dev)
        every = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(every, mine)
        cyc = torch.stack(every).cpu().numpy()
        ep_allreduce = {"unit": "SM cycles of block 0, last layer call, per rank",
                        "own_partial_sums_stored": [int(v) for v in cyc[:, 0]],
                        "waiting_for_peer_flags": [int(v) for v in cyc[:, 1]],
                        "peer_parts_read_and_summed": [int(v) for v in cyc[:, 2]],
                        "kernel_us_per_launch": kernels.get("combine", {}).get("us_per_launch"),
                        "bytes_read_from_peers_per_rank": (world - 1) * B * N_MODEL * 4}

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
        del hws
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

    # ---- the CPU checker (rank 0): the reference's own CPU path where its library travelled with the
    # repository, else the scalar restatement
    oracle = ref = port = None
    if rank == 0 and not args.no_cpu:
        from oracle import oracle
        ref = oracle.ref()
        port = oracle.port()

    def cpu_layer(planar, x_np, ids_np, wts_np, gate_np):
        """One layer (routed experts + shared expert) on the CPU: planar [E + 1][blob]."""
        Bt = x_np.shape[0]
        if ref is not None:
            idh = np.concatenate([ids_np, np.full((Bt, 1), E, np.int32)], axis=1)
            gsig = (1.0 / (1.0 + np.exp(-gate_np.astype(np.float32)))).astype(np.float32)[:, None]
            wth = np.concatenate([wts_np, gsig], axis=1).astype(np.float32)
            return ref.moe_cpu(planar, EXPERT_BYTES, E + 1, N_MODEL, FF, x_np, idh, wth, workers=max(1, ref.physical_cpus()))
        return port.moe_layer(planar[:E], EXPERT_BYTES, planar[E], N_MODEL, FF, x_np, ids_np, wts_np, gate_np, n_threads=8)

    def parity_layer0(x_t, ids_t, wts_t, gate_t, out_t):
        """max |GPU - CPU| / RMS for layer 0 at the full shape (rank 0 only, else None)."""
        if rank != 0 or port is None or 0 not in keep:
            return None
        o = cpu_layer(keep[0], x_t.cpu().numpy(), ids_t.cpu().numpy(), wts_t.cpu().numpy(), gate_t.cpu().numpy())
        return rel_max(out_t.cpu().numpy(), o)

    # ---- CPU baseline: the reference's CPU path on a bounded sample (rank 0, single GPU runs only)
    cpu = None
    if rank == 0 and not args.no_cpu:
        if world == 1 and ref is not None:
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
                             f"as the GPU run), {sec * 1e3:.3f} ms per layer", "avx512_vnni": ref.have_avx512(),
                   "workers_sweep": cpu_workers_sweep(ref, planar, xs, idh, wth)}
        elif world == 1:
            cpu = {"value": None, "unit": UNIT, "cores": 0, "kind": "reference", "sample": "oracle/_ref not built"}
        else:
            cpu = {"value": None, "unit": UNIT, "cores": 0, "kind": "reference" if ref is not None else "port",
                   "sample": "not timed on a multi-GPU run (the single-GPU run carries the CPU timing); parity only"}
        # the GPU result against the CPU result on the same inputs, at every N
        cpu["gpu_vs_cpu_max_err_over_rms"] = parity_layer0(x[0], ids[0], wts[0], gate[0], out[0])

    if world > 1:   # every rank must hold the same routing and the same reduced output
        chk = torch.stack([out.double().sum(), ids.double().sum()])
        lo_, hi_ = chk.clone(), chk.clone()
        dist.all_reduce(lo_, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi_, op=dist.ReduceOp.MAX)
        assert torch.equal(lo_, hi_), "ranks disagree on the layer output"

    # ---- the other configurations, each with its own parity figure
    extra_steps = max(5, min(args.steps, 20))
    decode_batches, verify_stack, prefill = None, None, None
    if not args.no_extras:
        decode_batches = {}
        for Bs in (1, 4, 16):
            if Bs >= B:
                continue
            xs_, ls_, gs_ = x[:, :Bs].contiguous(), logits[:, :Bs].contiguous(), gate[:, :Bs].contiguous()
            ob = torch.empty(L, Bs, N_MODEL, device=dev)
            ib = torch.empty(L, Bs, K, dtype=torch.int32, device=dev)
            wb = torch.empty(L, Bs, K, device=dev)
            wsb = moe.workspace(moe.moe_layer_workspace_bytes(Bs, K, N_MODEL, FF), dev)

            def step_b():
                for l in range(L):
                    layer(l, xs_[l], ls_[l], gs_[l], ob[l], ib[l], wb[l], wsb)

            tb = timeit(step_b, 3, extra_steps)
            moe.workspace_status(wsb)
            db = [int(torch.unique(ib[l]).numel()) for l in range(L)]
            lb = layer_alg_bytes(db, Bs)
            decode_batches[str(Bs)] = {"us_per_layer": round(tb * 1e3 / L, 2), "value": round(Bs * L / (tb * 1e-3), 1), "unit": UNIT,
                                       "distinct_experts_per_layer_mean": float(np.mean(db)), "algorithmic_bytes_per_layer": int(lb),
                                       "frac_of_peak": round(lb / world / (tb * 1e-3 / L) / 1e9 / peak, 4),
                                       "parity_max_err_over_rms": parity_layer0(xs_[0], ib[0], wb[0], gs_[0], ob[0])}
            del wsb
        verify_stack = bench_verify_stack(torch, moe, synth, dev, rank, world, L, layer, timeit, layer_planar, x, logits, gate, port, peak,
                                          extra_steps)
        prefill = bench_prefill_extra(torch, dist, moe, synth, dev, rank, world, arena, e_lo, e_hi, keep, port, extra_steps, layer_planar)

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
            "roofline": roofline, "cpu_baseline": cpu, "decode_batches": decode_batches, "prefill": prefill, "verify_stack": verify_stack,
        }
        if ep_allreduce is not None:
            line["ep_allreduce"] = ep_allreduce
        print(json.dumps(line))
    if comm is not None:
        comm.close()
    if world > 1:
        dist.destroy_process_group()


def bench_verify_stack(torch, moe, synth, dev, rank, world, L, layer, timeit, layer_planar, x, logits, gate, port, peak, steps):
    """BASELINE configs[3]: the expert stack walked by a speculative-verify window of three tokens
    (1 + 2 drafts), the layers chained by x_next = rmsnorm_unit(x + y) in fp32, router logits
    pre-generated per layer; expert parallel when launched on several GPUs. The step is bound by
    48 x (five dependent kernels + the exchange), not by HBM: the fraction says how far."""
    T3 = 3
    ls_, gs_ = logits[:, :T3].contiguous(), gate[:, :T3].contiguous()
    xs = torch.empty(L + 1, T3, N_MODEL, device=dev)       # xs[l]: the input of layer l
    xs[0].copy_(x[0, :T3])
    ys = torch.empty(L, T3, N_MODEL, device=dev)
    ib = torch.empty(L, T3, K, dtype=torch.int32, device=dev)
    wb = torch.empty(L, T3, K, device=dev)
    wsb = moe.workspace(moe.moe_layer_workspace_bytes(T3, K, N_MODEL, FF), dev)

    def step():
        for l in range(L):
            layer(l, xs[l], ls_[l], gs_[l], ys[l], ib[l], wb[l], wsb)
            moe.chain_rmsnorm_unit(xs[l], ys[l], out=xs[l + 1])

    t = timeit(step, 3, steps)
    moe.workspace_status(wsb)
    db = [int(torch.unique(ib[l]).numel()) for l in range(L)]
    step_bytes = float(sum((d + 1) * EXPERT_BYTES for d in db))
    res = {"workload": f"configs[3]: {L} chained layers, {T3} tokens per step, 512 experts top-10 + shared, ep{world}",
           "value": round(T3 / (t * 1e-3), 1), "unit": "tokens/s", "ms_per_step": round(t, 4), "us_per_layer": round(t * 1e3 / L, 2),
           "algorithmic_bytes_per_step": int(step_bytes), "hbm_frac_of_peak": round(step_bytes / world / (t * 1e-3) / 1e9 / peak, 4),
           "note": "latency-limited: a layer is five dependent kernels (plus the exchange on several GPUs) over about 10 MB of weights"}
    if rank == 0 and port is not None:
        # Parity. The oracle needs only the experts the window uses: each layer's blobs are regenerated
        # on the device and the used ones copied out. Two figures: every layer's output against the
        # oracle's layer on the same input (and the join bit for bit), and the last layer's output
        # against the oracle run free over the whole chain.
        x_free = xs[0].cpu().numpy()
        worst, join_exact, ids_exact, y_free = 0.0, True, True, None
        for l in range(L):
            p = layer_planar(l)
            idl, wl, gl = ib[l].cpu().numpy(), wb[l].cpu().numpy(), gs_[l].cpu().numpy()
            uniq = np.unique(idl)
            sel = p[torch.from_numpy(np.append(uniq, E).astype(np.int64)).to(dev)].cpu().numpy()
            del p
            loc = np.searchsorted(uniq, idl).astype(np.int32)
            ids_exact = ids_exact and bool(np.array_equal(port.route(ls_[l].cpu().numpy(), K)[0], idl))
            x_l, y_l = xs[l].cpu().numpy(), ys[l].cpu().numpy()
            y_or = port.moe_layer(np.ascontiguousarray(sel[:-1]), EXPERT_BYTES, sel[-1], N_MODEL, FF, x_l, loc, wl, gl, n_threads=8)
            worst = max(worst, rel_max(y_l, y_or))
            join_exact = join_exact and bool(np.array_equal(port.chain_rmsnorm_unit(x_l, y_l), xs[l + 1].cpu().numpy()))
            y_free = port.moe_layer(np.ascontiguousarray(sel[:-1]), EXPERT_BYTES, sel[-1], N_MODEL, FF, x_free, loc, wl, gl, n_threads=8)
            x_free = port.chain_rmsnorm_unit(x_free, y_free)
        res["parity"] = {"per_layer_max_err_over_rms": worst, "layer_join_bit_exact": join_exact, "router_ids_bit_exact": ids_exact,
                         "last_layer_free_running_err_over_rms": rel_max(ys[L - 1].cpu().numpy(), y_free),
                         "checker": "scalar restatement of the reference's CPU path, every layer"}
    return res


def bench_prefill_extra(torch, dist, moe, synth, dev, rank, world, arena, e_lo, e_hi, keep, port, steps, layer_planar):
    """BASELINE configs[2] (one GPU: 4,096 tokens, Zipf routing) or configs[4] (several GPUs: 16,384
    tokens, uniform and Zipf routing, tokens and experts sharded, all-to-all dispatch and combine)
    on the experts of layer 0. A step is route + grouped expert products + combine."""
    from flashrt_b200 import ep
    peak_tf = 1657.0
    pk = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(pk):
        peak_tf = float(json.load(open(pk))["bf16_tflops"])
    T = 4096 if world == 1 else 16384
    Tl = T // world
    res = {}
    for routing in (("zipf",) if world == 1 else ("uniform", "zipf")):
        xa = synth.activations(T, N_MODEL, through_bf16=True)
        la = synth.zipf_logits(T, E) if routing == "zipf" else synth.router_logits(T, E)
        x = torch.from_numpy(xa[rank * Tl:(rank + 1) * Tl]).to(dev)
        lg = torch.from_numpy(la[rank * Tl:(rank + 1) * Tl]).to(dev)
        keepers = {}
        if world == 1:
            ws = moe.workspace(moe.moe_q2.workspace_bytes(T, K, N_MODEL, FF, E), dev)
            yd = torch.empty(T * K, N_MODEL, device=dev)
            out = torch.empty(T, N_MODEL, device=dev)

            def step():
                ids, wts = moe.moe_route_topk(lg, K)
                moe.moe_q2.run(arena.blob(0, 0), arena.stride, E, N_MODEL, FF, x, ids, yd=yd, ws=ws)
                moe.moe_combine(yd.view(T, K, N_MODEL), wts, None, None, None, out=out)
                keepers["ids"], keepers["wts"] = ids, wts
        else:
            # Skewed routing: the experts are dealt to the ranks round-robin in order of popularity (a
            # load-time decision: the counts of one routing pass over the tokens), uniform routing keeps
            # contiguous ranges. A dealt placement gets its own arena, loaded with this rank's experts.
            owner, ptr, stride_ = None, arena.blob(0, 0), arena.stride
            if routing == "zipf":
                top = torch.topk(torch.from_numpy(la).to(dev), K, dim=1).indices
                counts = torch.bincount(top.reshape(-1), minlength=E).cpu().numpy()
                owner = ep.expert_placement(counts, world)
                mine = np.nonzero(owner == rank)[0]
                keepers["arena"] = moe.ExpertArena(1, len(mine), N_MODEL, FF)
                p0 = layer_planar(0)
                keepers["arena"].load_planar(0, 0, len(mine), p0[torch.from_numpy(mine).to(dev)].contiguous().view(-1))
                del p0
                ptr, stride_ = keepers["arena"].blob(0, 0), keepers["arena"].stride
            pipe = ep.PrefillEp(ptr, stride_, E, N_MODEL, FF, Tl, K, owner=owner)

            def step():
                keepers["out"], keepers["ids"], keepers["wts"] = pipe.run(x, lg)

        for _ in range(2):
            step()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            step()
        b.record()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        ms = a.elapsed_time(b) / steps
        if world > 1:
            tt = torch.tensor([ms], device=dev)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            ms = float(tt.item())
        ncls = 16
        pms, pn = (C.c_float * ncls)(), (C.c_int * ncls)()
        moe.check(moe.lib.frx_profile_begin())
        step()
        moe.check(moe.lib.frx_profile_end(pms, pn, ncls))
        names = [moe.lib.frx_profile_class_name(i).decode() for i in range(ncls)]
        kus = {names[i]: round(1e3 * float(pms[i]), 2) for i in range(ncls) if pn[i]}
        flops = T * K * 3 * 2 * N_MODEL * FF
        gemm_ms = (kus.get("gate_up", 0.0) + kus.get("down", 0.0)) / 1e3
        ids_all = keepers["ids"]
        cnt = torch.bincount(ids_all.reshape(-1).to(torch.int64), minlength=E)
        entry = {"workload": f"configs[{2 if world == 1 else 4}]: one MoE layer prefill, {T} tokens, hidden 2048, 512 experts top-10, "
                             f"{routing} routing, ep{world}",
                 "value": round(T / (ms * 1e-3), 1), "unit": "tokens/s", "ms_per_step": round(ms, 4), "kernels_us": kus,
                 "flops_per_step": flops, "tflops_step": round(flops / (ms * 1e-3) / 1e12, 1),
                 "tflops_expert_products_rank0": round(flops / world / max(gemm_ms, 1e-9) / 1e9, 1) if gemm_ms else None,
                 "frac_of_bf16_peak_step": round(flops / world / (ms * 1e-3) / 1e12 / peak_tf, 4), "peak_tflops": peak_tf,
                 "form": ("tcgen05" if T * K >= 256 * E else "streaming") if world == 1
                 else "streaming per chunk of 4 (slots per expert and chunk below 256); Q8 all-gather dispatch, fp32 reduce-scatter combine, "
                      + ("experts dealt round-robin by popularity" if routing == "zipf" else "contiguous expert ranges"),
                 "tokens_per_expert_rank0": {"mean": float(cnt.float().mean()), "max": int(cnt.max()), "min": int(cnt.min())}}
        if rank == 0 and port is not None and 0 in keep:
            ids_np, wts_np = ids_all.cpu().numpy(), keepers["wts"].cpu().numpy()
            xl = xa[:Tl]
            ids_or, _, _ = port.route(la[:64], K)
            entry["router_ids_bit_exact_64_tokens"] = bool(np.array_equal(ids_or, ids_np[:64]))
            xq, xd = port.quantize_q8(xl[:8])
            if world == 1:
                ys = yd.view(T, K, N_MODEL)
                worst = 0.0
                rng = np.random.default_rng(1)
                for t_, k_ in zip(rng.integers(0, 8, 12), rng.integers(0, K, 12)):
                    want = port.expert_ffn(keep[0][ids_np[t_, k_]], N_MODEL, FF, xq[t_], xd[t_])
                    worst = max(worst, rel_max(ys[t_, k_].cpu().numpy(), want))
                entry["parity_slot_sample_max_err_over_rms"] = worst
                got = out[:2].cpu().numpy()
            else:
                got = keepers["out"][:2].cpu().numpy()
            want = np.stack([port.moe_layer(np.ascontiguousarray(keep[0][np.sort(ids_np[t_])]), EXPERT_BYTES, None, N_MODEL, FF, xl[t_:t_ + 1],
                                            np.arange(K, dtype=np.int32)[None], wts_np[t_:t_ + 1][:, np.argsort(ids_np[t_])], None)[0]
                             for t_ in range(2)])
            entry["parity_layer_output_2_tokens_max_err_over_rms"] = rel_max(got, want)
        res[routing] = entry
        if world == 1:
            del ws, yd, out
    return res


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

    pipe = ep.PrefillEp(arena.blob(0, 0), arena.stride, E, N_MODEL, FF, Tl, K) if world > 1 else None

    def step():
        if world == 1:
            ids, wts = moe.moe_route_topk(logits, K)
            moe.moe_q2.run(arena.blob(0, 0), arena.stride, E, N_MODEL, FF, x, ids, yd=yd, ws=ws, form=args.form)
            moe.moe_combine(yd.view(Tl, K, N_MODEL), wts, None, None, None, out=out)
        else:
            pipe.run(x, logits)

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
    ncls = 16
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
    ap.add_argument("--no-extras", action="store_true", help="headline only: skip the decode_batches, prefill and verify_stack keys")
    ap.add_argument("--nw", type=int, default=0, help="tuning: consumer warps of the streaming kernel (8, 12, 16, 20)")
    ap.add_argument("--fused", type=int, default=None, help="tuning: 0 runs the decode FFN as three kernels instead of one")
    ap.add_argument("--deal-shared", type=int, default=1, help="expert parallel: 1 deals the shared expert's tokens among the ranks, 0 leaves them all to rank 0")
    ap.add_argument("--down-weight", type=int, default=None, help="tuning: weight (in 1/16) of a down task of a 3-4 token item in the split over blocks; 0 = even split")
    ap.add_argument("--evict-first", type=int, default=None, help="tuning: 0 copies the decode layer's weights with the default L2 policy")
    ap.add_argument("--down-item-weight", type=int, default=None, help="tuning: weight (in 1/16 of a task) of an item's buffer in down's split over blocks")
    ap.add_argument("--small-limits", default=None, help="tuning: tasks per SM up to which blocks of 4 and of 8 warps are used, e.g. 4,8 (default) or 0,0")
    ap.add_argument("--fold", type=int, default=None, help="tuning: 0 runs the hidden-row quantizer as its own kernel")
    ap.add_argument("--ffn-buffers", default=None, help="tuning: item buffers of the fused FFN kernel, gate/up,down (e.g. 3,3)")
    ap.add_argument("--task4", type=int, default=None, help="tuning: 0 keeps two row groups per task in the decode layer")
    ap.add_argument("--gu-chunks", type=int, default=0, help="tuning: K slices per gate/up task")
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
