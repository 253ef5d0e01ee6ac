#!/usr/bin/env python
"""Throughput of the INT4 MoE layer on B200, with its roofline fraction and a CPU baseline.

Headline workload (config.workload): one Gemma-4-26B-A4B-shaped MoE layer at decode — one token
[1 x 2816] through router top-8, eight INT4 GeGLU experts out of 128 and the shared INT4 FFN.
A "step" is one token through one layer.  Steps rotate over several resident layers and input
rows so that a step's 37.5 MB of weights cannot be served from L2 by the previous step.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

For N > 1 (launched under torch.distributed.run) every rank runs an independent replica of the
workload on its own GPU — decode does not shard — and the value is the sum over ranks divided by
the slowest rank's device time.  `--impl reference` times the reference's CPU path (this
repository's C restatement of it, since the Swift/Metal code cannot run on Linux) on the host
cores, rank 0 only.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

D, F, FS, E, K = 2816, 704, 2112, 128, 8
EXPERT_BYTES = 3 * (F * D // 2 + 2 * (F * D // 64) * 2)          # 3 345 408
SHARED_BYTES = 3 * (FS * D // 2 + 2 * (FS * D // 64) * 2)        # 10 036 224
ROUTER_BYTES = E * D * 2                                         # 720 896
ACT_IO_BYTES = 2 * D * 2                                         # x in, y out
DECODE_BYTES = K * EXPERT_BYTES + SHARED_BYTES + ROUTER_BYTES + ACT_IO_BYTES  # 37 531 648
DECODE_FLOPS = 2 * (K * 3 * F * D + 3 * FS * D + E * D)
ROOT_SEED = 0xF1E1DFA2E
MIN_TIMED_SECONDS = 0.25  # every leg's timed region runs at least this long
DECODE_PROFILE = os.path.join("profiles", "decode_fused_config1.md")


def profiled_decode_traffic():
    """dram__bytes_read.sum + dram__bytes_write.sum of one decode launch, as recorded in the ncu
    summary under profiles/ — only when that summary was taken from the kernel sources that are
    being run (it records their SHA-256); otherwise None: a stale capture is not reported."""
    import hashlib
    import re
    path = os.path.join(ROOT, DECODE_PROFILE)
    if not os.path.exists(path):
        return None, "no profile"
    text = open(path).read()
    h = hashlib.sha256()
    for name in ("ff_decode.cu", "ff_mma_device.cuh"):
        with open(os.path.join(ROOT, "ane_fieldfare_b200", "csrc", name), "rb") as fh:
            h.update(fh.read())
    digest = re.search(r"kernel sources sha256: ([0-9a-f]{64})", text)
    traffic = re.search(r"traffic bytes per launch: (\d+)", text)
    if not digest or not traffic:
        return None, "profile records no source hash"
    if digest.group(1) != h.hexdigest():
        return None, f"{DECODE_PROFILE} was captured from other kernel sources"
    return int(traffic.group(1)), DECODE_PROFILE


PREFILL_TOKENS = 4096


def measured_bf16_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            p = json.load(fh)
        return {"tflops": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])),
                "burst_tflops": float(p["bf16_tflops"]), "source": "measured (sustained)"}
    return {"tflops": 1400.0, "burst_tflops": 1590.0, "source": "fallback"}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            p = json.load(fh)
        return {"hbm_gbs": float(p["hbm_gbs"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}",
                 "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
            deadline = time.time() + 3.0
            while not self.lines and time.time() < deadline:
                time.sleep(0.02)
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                smax.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None,
                "sm_max_mhz": max(smax) if smax else None, "reasons": sorted(reasons),
                "samples": len(sm)}


def dist_env():
    return (int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0")),
            int(os.environ.get("WORLD_SIZE", "1")))


def cpu_decode_baseline(layer_host, tokens_bits, seconds_budget=12.0, max_steps=None):
    """Times the CPU oracle's decode layer (all host threads) on a bounded sample of steps."""
    from oracle import oracle as O
    O.set_num_threads(os.cpu_count() or 1)
    ld = O.LayerData(experts=layer_host.blobs, stride=layer_host.layout.stride,
                     off=layer_host.layout.offsets.as_tuple(), E=E, D=D, F=F, K=K,
                     shared=layer_host.sharedBlob, shared_off=layer_host.sharedLayout.offsets.as_tuple(),
                     Fs=FS, router_w=layer_host.routerW, logit_bias=layer_host.logitBias)
    O.moe_layer(ld, tokens_bits[:1], O.MODE_DECODE)  # warm
    steps, t0 = 0, time.perf_counter()
    while True:
        row = tokens_bits[steps % len(tokens_bits)][None, :]
        O.moe_layer(ld, row, O.MODE_DECODE)
        steps += 1
        elapsed = time.perf_counter() - t0
        if (max_steps and steps >= max_steps) or (not max_steps and elapsed > seconds_budget):
            break
    return steps / elapsed, steps, O.num_threads()


def run_reference(args):
    """The reference arm: the CPU restatement of the reference's decode path on the host cores."""
    rank, _, world = dist_env()
    if rank != 0:
        return
    from ane_fieldfare_b200 import workload
    layer = workload.make_layer(ROOT_SEED, 0)
    tokens = workload.make_tokens(ROOT_SEED, "decode.x", 64, D)
    for _ in range(max(args.warmup, 1)):
        cpu_decode_baseline(layer, tokens, max_steps=1)
    rate, steps, threads = cpu_decode_baseline(layer, tokens, max_steps=args.steps)
    line = {
        "impl": "reference", "metric": "int4_moe_layer_tokens_per_s", "value": rate,
        "unit": "tokens/s", "n_gpus": args.gpus, "steps": steps, "warmup": args.warmup,
        "ms_per_step": 1e3 / rate, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int4 weights, bf16 activations, fp32 accumulate", "data": "synthetic",
        "config": {"workload": "config1_decode_1token_moe_layer", "hidden": D, "experts": E,
                   "top_k": K, "expert_intermediate": F, "shared_intermediate": FS},
        "cpu_baseline": {"value": rate, "unit": "tokens/s", "cores": threads, "kind": "port",
                         "sample": f"{steps} decode steps of the C oracle (OpenMP), one layer"},
        "e2e": {"value": rate, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    emit(line)


def time_graph(torch, stream, graph, replays):
    """Device time of `replays` graph launches, CUDA events on the launching stream."""
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream):
        begin.record(stream)
        for _ in range(replays):
            graph.replay()
        end.record(stream)
        stream.synchronize()
    return begin.elapsed_time(end)


def time_replays(torch, stream, launch, replays):
    """Milliseconds of each of `replays` back-to-back calls of launch(), from CUDA events recorded
    between them on the launching stream (no host synchronisation inside the region)."""
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(replays + 1)]
    with torch.cuda.stream(stream):
        marks[0].record(stream)
        for i in range(replays):
            launch()
            marks[i + 1].record(stream)
        stream.synchronize()
    return [marks[i].elapsed_time(marks[i + 1]) for i in range(replays)]


def spread(per_replay_ms, steps_per_replay):
    a = np.asarray(per_replay_ms, dtype=np.float64) / steps_per_replay
    return {"replays": int(a.size), "steps_per_replay": int(steps_per_replay), "total_ms": float(a.sum() * steps_per_replay),
            "median_us_per_step": float(np.median(a) * 1e3), "min_us_per_step": float(a.min() * 1e3),
            "max_us_per_step": float(a.max() * 1e3)}


def capture_steps(torch, ctx, stream, step, group):
    """One CUDA graph holding `group` consecutive steps (a few uncaptured steps run first so that
    every kernel is configured before the capture).  Returns the graph and the number of kernels
    the library enqueued per step while capturing."""
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        for i in range(3):
            step(i)
        stream.synchronize()
        before = ctx.info().kernelLaunches
        with torch.cuda.graph(graph, stream=stream):
            for i in range(group):
                step(i)
        launched = ctx.info().kernelLaunches - before
    return graph, launched / group


def traced_kernels(ctx, step, group):
    """Per-kernel device time of `group` steps by CUDA events (outside any graph)."""
    ctx.setTracing(True)
    for i in range(group):
        step(i)
    trace = ctx.trace()
    ctx.setTracing(False)
    return {name: {"launches": n, "avg_us": round(1e3 * t / n, 3)} for name, (n, t) in trace.items()}


STACK_DISTINCT_LAYERS = 3
STACK_LAYERS = 30
STACK_TOKENS = 32768


def stack_flops(layers):
    return layers * STACK_TOKENS * (2 * (K * 3 * F * D + 3 * FS * D + E * D))


def measure_stack_single(torch, hotpath, workload, host_layers, local_rank, device, args):
    """Configuration 4 on one GPU: all experts of all layers resident in one context, the stack run
    by the library's own ff_moe_stack (RMSNorm + block per layer) — the time the expert-parallel
    runs are compared with."""
    from ane_fieldfare_b200 import synth
    layers = args.stack_layers
    ctx = hotpath.HotpathContext(layers=layers, experts=E, d=D, f=F, sharedF=FS, topK=K,
                                 maxTokens=STACK_TOKENS, device=local_rank)
    for slot in range(layers):
        L = host_layers[slot % len(host_layers)]
        ctx.loadLayer(slot, L.blobs, L.layout.stride, L.layout.offsets)
        ctx.loadShared(slot, *L.shared_projections())
        ctx.loadRouter(slot, L.routerW,
                       logitBias=synth.zipf_log_prior(E, 1.1, ROOT_SEED, f"stack.zipf.{slot % len(host_layers)}"))
    x0 = hotpath.bf16_tensor(workload.make_tokens(ROOT_SEED, "stack.x", STACK_TOKENS, D), device)
    y = torch.empty_like(x0)
    for _ in range(2):
        ctx.moeStack(0, layers, x0, 1e-6, y)
    torch.cuda.synchronize()
    steps = 3
    per = time_replays(torch, torch.cuda.current_stream(), lambda: ctx.moeStack(0, layers, x0, 1e-6, y), steps)
    ms = float(np.median(per))
    ctx.setTracing(True)
    ctx.moeStack(0, layers, x0, 1e-6, y)
    trace = ctx.trace()
    ctx.setTracing(False)
    finite = bool(torch.isfinite(y.float()).all().item())
    err = ctx.info().deviceErrorFlag
    resident = ctx.info().weightBytesResident
    ctx.close()
    peak = measured_bf16_peak()
    tf = stack_flops(layers) / (ms * 1e-3) / 1e12
    return {"workload": f"config4_stack_{layers}layers_{STACK_TOKENS}tokens", "gpus": 1,
            "path": "ff_moe_stack on one context (no expert parallelism, no collective)",
            "tokens_per_s": STACK_TOKENS / (ms * 1e-3), "ms_per_stack": ms, "steps": steps,
            "timed_region": spread(per, 1), "tflops": tf,
            "frac_of_measured_bf16_sustained": tf / peak["tflops"], "frac_of_measured_bf16_burst": tf / peak["burst_tflops"],
            "weight_bytes_resident": int(resident), "output_finite": finite, "device_error_flag": int(err),
            "kernel_ms_per_stack": {name: round(t, 3) for name, (n, t) in sorted(trace.items())}}


def measure_stack(torch, dist, hotpath, workload, host_layers, rank, local_rank, world, device, args):
    """Benchmark configuration 4: a 30-layer stack of MoE blocks (RMSNorm between layers, no
    attention), 32768 prefill tokens.  One GPU: the library's ff_moe_stack.  Several GPUs: experts
    sharded over the ranks with an NCCL all-to-all dispatch and combine per layer.  All 30 layer
    slots are resident (13.2 GB over the box); their bytes repeat a few distinct seeded layers,
    which does not change the work."""
    from ane_fieldfare_b200 import parallel, synth
    if world == 1:
        return measure_stack_single(torch, hotpath, workload, host_layers, local_rank, device, args)
    layers = args.stack_layers
    tokens_local = STACK_TOKENS // world
    epr = E // world
    capacity = min(STACK_TOKENS * K, 4 * tokens_local * K)
    home = hotpath.HotpathContext(layers=len(host_layers), experts=E, d=D, f=F, sharedF=FS, topK=K,
                                  maxTokens=tokens_local, device=local_rank)
    local = hotpath.HotpathContext(layers=layers, experts=epr, d=D, f=F, sharedF=0, topK=1,
                                   maxTokens=capacity, device=local_rank)
    # the same experts behind a context that takes K routes per row: for the exchange that sends a
    # token's row once per destination rank
    local_k = None
    if args.ep_comm in ("peer", "both"):
        local_k = hotpath.HotpathContext(layers=layers, experts=epr, d=D, f=F, sharedF=0, topK=K,
                                         maxTokens=STACK_TOKENS, device=local_rank)
    for i, L in enumerate(host_layers):
        home.loadShared(i, *L.shared_projections())
        home.loadRouter(i, L.routerW, logitBias=synth.zipf_log_prior(E, 1.1, ROOT_SEED, f"stack.zipf.{i}"))

    def load_experts(placements):
        for slot in range(layers):
            L = host_layers[slot % len(host_layers)]
            mine = placements[slot].experts_of(rank)
            blobs = np.ascontiguousarray(L.blobs[mine])
            local.loadLayer(slot, blobs, L.layout.stride, L.layout.offsets, expertCount=epr)
            if local_k is not None and placements[slot].rank_of is not contiguous[slot].rank_of:
                local_k.loadLayer(slot, blobs, L.layout.stride, L.layout.offsets, expertCount=epr)

    sorter = parallel.cuda_route_sorter(home)

    def make_blocks(placements, chunks, peer=None, one_row_per_token=False):
        out = []
        for slot in range(layers):
            # the home context is indexed by the distinct layer, the expert context by the stack's slot
            fns = parallel.cuda_layer_fns(home, local_k if one_row_per_token else local, slot % len(host_layers),
                                          expert_layer=slot)
            out.append(parallel.ExpertParallelMoE(E, K, *fns, placement=placements[slot], chunks=chunks, peer=peer,
                                                  one_row_per_token=one_row_per_token, route_sorter=sorter))
        return out

    x0 = hotpath.bf16_tensor(workload.make_tokens(ROOT_SEED + rank, "stack.x", tokens_local, D), device)

    def run_stack(blocks):
        x = x0
        for block in blocks:
            x = block.forward(home.rmsnorm(x, None, 1e-6))
        return x

    # Pass 1, contiguous placement: the stack's outputs do not depend on where an expert lives, so
    # this pass measures how many routes every expert of every layer receives (summed over the
    # ranks).  Experts are then placed so that every rank receives about the same number of rows
    # (the blob layout is untouched: a rank loads the blobs of its experts).
    contiguous = [parallel.contiguous_placement(E, world)] * layers
    load_experts(contiguous)  # (the K-wide expert context is loaded with the final placement only)
    blocks = make_blocks(contiguous, 1)
    for block in blocks:
        block.count_experts = True
    run_stack(blocks)
    counts = torch.stack([block.last_expert_counts for block in blocks]).to(torch.float64)
    dist.all_reduce(counts)
    placements = [parallel.balanced_placement((counts[slot] + 0.5).tolist(), world) for slot in range(layers)]
    load_experts(placements)
    # two ways to move the rows: the collective (tokens in chunks whose exchanges overlap the GEMMs)
    # and peer stores into symmetric memory; both are checked and timed, the faster one is the line
    variants = {"nccl_all_to_all": make_blocks(placements, args.ep_chunks)}
    if args.ep_chunks != 1:
        variants["nccl_all_to_all_unchunked"] = make_blocks(placements, 1)
    peer_note = None
    if args.ep_comm in ("peer", "both"):
        ok = torch.ones(1, dtype=torch.float64, device=device)
        try:
            buffers = parallel.PeerBuffers(capacity, D, torch.bfloat16, device)
            buffers_k = parallel.PeerBuffers(capacity, D, torch.bfloat16, device, ids_width=K)
        except Exception as exc:  # symmetric memory not available on this box
            peer_note = f"{type(exc).__name__}: {exc}"[:200]
            ok.zero_()
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if ok.item() == 1.0:
            variants["peer_stores"] = make_blocks(placements, 1, peer=buffers)
            variants["peer_stores_one_row_per_token_and_rank"] = make_blocks(placements, 1, peer=buffers_k,
                                                                             one_row_per_token=True)
        if args.ep_comm == "peer" and "peer_stores" in variants:
            variants.pop("nccl_all_to_all", None)
            variants.pop("nccl_all_to_all_unchunked", None)

    # the first layer's output for the first rows against ff_moe_layer on one context that holds all
    # experts of that layer: the same bits
    check_rows = min(256, tokens_local)
    full = hotpath.HotpathContext(layers=1, experts=E, d=D, f=F, sharedF=FS, topK=K, maxTokens=tokens_local,
                                  device=local_rank)
    L0 = host_layers[0]
    workload.load_layer(full, 0, L0)
    full.loadRouter(0, L0.routerW, logitBias=synth.zipf_log_prior(E, 1.1, ROOT_SEED, "stack.zipf.0"))
    normed = home.rmsnorm(x0, None, 1e-6)
    y_one = full.moeLayer(0, normed)
    same = torch.ones(1, dtype=torch.float64, device=device)
    for blocks in variants.values():
        y_ep = blocks[0].forward(normed)
        torch.cuda.synchronize()
        if not torch.equal(y_ep[:check_rows], y_one[:check_rows]):
            same.zero_()
    full.close()
    dist.all_reduce(same, op=dist.ReduceOp.MIN)

    steps = 3
    results = {}
    for name, blocks in variants.items():
        for _ in range(2):
            run_stack(blocks)
        torch.cuda.synchronize()
        dist.barrier()
        per = time_replays(torch, torch.cuda.current_stream(), lambda: run_stack(blocks), steps)
        t = torch.tensor([float(np.median(per))], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        # one more pass with CUDA events around the phases of every layer
        timer = parallel.PhaseTimer()
        for block in blocks:
            block.timer = timer
        y = run_stack(blocks)
        phases = timer.totals()
        names = sorted(phases)
        pt = torch.tensor([phases[n] for n in names], dtype=torch.float64, device=device)
        dist.all_reduce(pt, op=dist.ReduceOp.MAX)
        results[name] = {"ms_per_stack": float(t.item()),
                         "phase_ms_per_stack_max_over_ranks": {n: round(float(v), 3) for n, v in zip(names, pt.tolist())}}
    best = min(results, key=lambda n: results[n]["ms_per_stack"])
    ms = results[best]["ms_per_stack"]
    blocks = variants[best]
    recv = torch.tensor([[float(b.last_recv_rows) for b in blocks]], dtype=torch.float64, device=device)
    rows = [torch.zeros_like(recv) for _ in range(world)]
    dist.all_gather(rows, recv)
    rows = torch.cat(rows).cpu().numpy()  # [world, layers]
    finite = bool(torch.isfinite(y.float()).all().item())
    err = home.info().deviceErrorFlag | local.info().deviceErrorFlag | (local_k.info().deviceErrorFlag if local_k else 0)
    peak = measured_bf16_peak()
    home.close()
    local.close()
    if local_k is not None:
        local_k.close()
    tf = stack_flops(layers) / (ms * 1e-3) / 1e12
    return {"workload": f"config4_stack_{layers}layers_{STACK_TOKENS}tokens_expert_parallel", "gpus": world,
            "tokens_per_s": STACK_TOKENS / (ms * 1e-3), "ms_per_stack": ms, "steps": steps,
            "tflops": tf, "frac_of_measured_bf16_sustained_per_gpu": tf / (peak["tflops"] * world),
            "ep_matches_single_gpu": bool(same.item() == 1.0),
            "ep_check": f"layer 0, first {check_rows} local rows of every rank, bitwise against ff_moe_layer "
                        "on one context holding all 128 experts",
            "exchange": best, "exchanges_measured": results, "peer_stores_unavailable": peer_note,
            "rows_received_per_rank_by_layer": rows.astype(np.int64).T.tolist(),
            "rows_received_max_over_mean": float((rows.max(axis=0) / rows.mean(axis=0)).mean()),
            "chunks_per_layer": args.ep_chunks,
            "output_finite": finite, "device_error_flag": int(err),
            "exchange_kinds": {"nccl_all_to_all": "all_to_all_single for dispatch and combine of every layer and chunk, "
                                                  "asynchronous to the GEMMs",
                               "nccl_all_to_all_unchunked": "the same with the local tokens in one run",
                               "peer_stores": "rows gathered and copied straight into the destination rank's buffer in "
                                              "symmetric memory over NVLink, a barrier across the ranks after each",
                               "peer_stores_one_row_per_token_and_rank": "the same, a token's row sent once to every rank "
                                              "that holds any of its experts, with its K-wide list of local expert ids"},
            "placement": "experts assigned to ranks by greedy balancing of the routes each expert of each layer "
                         "received in a first pass of the same stack"}


def oracle_layer_data(O, layer_host, logit_bias):
    return O.LayerData(experts=layer_host.blobs, stride=layer_host.layout.stride,
                       off=layer_host.layout.offsets.as_tuple(), E=E, D=D, F=F, K=K,
                       shared=layer_host.sharedBlob, shared_off=layer_host.sharedLayout.offsets.as_tuple(),
                       Fs=FS, router_w=layer_host.routerW, logit_bias=logit_bias)


def cpu_other_configs(layer_host, bias_verify, bias_prefill):
    """The CPU oracle on bounded samples of configurations 0, 2 and 3 (tokens per second each)."""
    from ane_fieldfare_b200 import workload
    from oracle import oracle as O
    O.set_num_threads(os.cpu_count() or 1)
    out = {}

    def timed(fn, tokens, budget, what):
        fn()
        n, t0 = 0, time.perf_counter()
        while n == 0 or time.perf_counter() - t0 < budget:
            fn()
            n += 1
        dt = time.perf_counter() - t0
        return {"value": tokens * n / dt, "unit": "tokens/s", "sample": f"{n} x {what}", "seconds": dt}

    x1 = workload.make_tokens(ROOT_SEED, "cfg0.x", 1, D)
    off = layer_host.layout.offsets.as_tuple()
    out["config0_single_expert_1token"] = timed(
        lambda: O.expert_ffn(layer_host.blobs[0], off, D, F, x1), 1, 2.0, "one expert, one token")
    x16 = workload.make_tokens(ROOT_SEED, "verify.x", 16, D)
    ld2 = oracle_layer_data(O, layer_host, bias_verify)
    out["config2_verify_16token_block"] = timed(
        lambda: O.moe_layer(ld2, x16, O.MODE_PARTIALS), 16, 4.0, "16-token block, one layer")
    x256 = workload.make_tokens(ROOT_SEED, "prefill.x", 256, D)
    ld3 = oracle_layer_data(O, layer_host, bias_prefill)
    out["config3_prefill_zipf"] = timed(
        lambda: O.moe_layer(ld3, x256, O.MODE_PARTIALS), 256, 6.0,
        "the first 256 of the 4096 tokens, one layer (tokens/s extrapolates linearly)")
    return out


def run_ours(args):
    import torch
    import torch.distributed as dist
    from ane_fieldfare_b200 import hotpath, synth, workload

    rank, local_rank, world = dist_env()
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    n_layers = args.layers
    want = set(args.only.split(",")) if args.only else {"decode", "verify", "prefill", "stack"}
    max_tokens = PREFILL_TOKENS if "prefill" in want else 16
    ctx = hotpath.HotpathContext(layers=n_layers, experts=E, d=D, f=F, sharedF=FS, topK=K,
                                 maxTokens=max_tokens, device=local_rank)
    host_layers = []
    for slot in range(n_layers):
        L = workload.make_layer(ROOT_SEED, slot)
        workload.load_layer(ctx, slot, L)
        host_layers.append(L if slot < STACK_DISTINCT_LAYERS else (L.routerW,))
    host_layer0 = host_layers[0]
    peaks = measured_peaks()
    stream = torch.cuda.Stream(device=device)
    min_s = 0.0 if args.quick else MIN_TIMED_SECONDS

    def router_bias(kind, slot):
        if kind == "none":
            return None
        if kind == "normal":
            return synth.normal(synth.seedtree_key(ROOT_SEED, f"bench.bias.{slot}"), E).astype(np.float32)
        return synth.zipf_log_prior(E, 1.1, ROOT_SEED, f"bench.zipf.{slot}")

    def set_router_bias(kind):
        for slot in range(n_layers):
            router = host_layers[slot].routerW if slot < STACK_DISTINCT_LAYERS else host_layers[slot][0]
            ctx.loadRouter(slot, router, logitBias=router_bias(kind, slot))

    def sync_max(ms):
        if world > 1:
            t = torch.tensor([ms], dtype=torch.float64, device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item())
        return ms

    def measure_graph(step, group, warm_steps, all_ranks=True):
        """Captures `group` consecutive steps as one CUDA graph, replays it until the timed region
        has run for MIN_TIMED_SECONDS, and returns (median ms of one replay as the max over ranks,
        spread record, kernels per step, clock record).  all_ranks: every rank runs this leg (then
        the ranks meet at barriers and the time is the maximum over them); a leg that rank 0 runs
        alone must not touch a collective."""
        graph, per_step = capture_steps(torch, ctx, stream, step, group)
        est = time_graph(torch, stream, graph, max(1, (warm_steps + group - 1) // group))
        est = max(est / max(1, (warm_steps + group - 1) // group), 1e-3)
        replays = max(3, int(np.ceil(min_s * 1e3 / est)))
        if world > 1 and all_ranks:
            dist.barrier()
        torch.cuda.synchronize()
        sampler = ClockSampler(local_rank)
        if rank == 0:
            sampler.start()
        per_replay = time_replays(torch, stream, graph.replay, replays)
        torch.cuda.synchronize()
        clocks = sampler.stop() if rank == 0 else None
        if world > 1 and all_ranks:
            dist.barrier()
        ms_replay = float(np.median(per_replay))
        return (sync_max(ms_replay) if all_ranks else ms_replay), spread(per_replay, group), per_step, clocks

    line = {}
    # ================= decode: config 1, the headline =================
    n_rows = 64
    tokens_bits = workload.make_tokens(ROOT_SEED, "decode.x", n_rows, D)
    x_rows = hotpath.bf16_tensor(tokens_bits, device)
    xs = [x_rows[i:i + 1].contiguous() for i in range(n_rows)]
    y1 = torch.zeros((1, D), dtype=torch.bfloat16, device=device)

    def decode_step(i):
        ctx.moeLayer(i % n_layers, xs[i % n_rows], y1)

    set_router_bias("none")
    warmup = max(args.warmup, 3)
    for i in range(warmup):
        decode_step(i)
    torch.cuda.synchronize()
    steps = max(1, min(args.steps, 8192))  # one CUDA graph holds exactly these steps
    ms, timing, kernels_per_step, clocks = measure_graph(decode_step, steps, warmup)
    value = world * steps / (ms * 1e-3)
    kernels = {"decode_fused": {"launches_per_step": kernels_per_step,
                                "avg_us_in_graph": round(1e3 * ms / steps / max(kernels_per_step, 1), 3)}}
    if not args.quick:
        eager = traced_kernels(ctx, decode_step, n_layers * 8)
        for name, rec in eager.items():
            kernels.setdefault(name, {})["avg_us_eager_with_launch_gaps"] = rec["avg_us"]

    # end to end through the host-buffer entry point
    hx = [torch.from_numpy(tokens_bits[i:i + 1].view(np.int16).copy()).view(torch.bfloat16).pin_memory()
          for i in range(n_rows)]
    hy = torch.zeros((1, D), dtype=torch.bfloat16).pin_memory()
    for i in range(5):
        ctx.moeLayerHost(i % n_layers, hx[i % n_rows], hy)
    e2e_steps = 8 if args.quick else max(steps, 6000)
    if world > 1:
        dist.barrier()
    t0 = time.perf_counter()
    for i in range(e2e_steps):
        ctx.moeLayerHost(i % n_layers, hx[i % n_rows], hy)
    e2e_s = sync_max(time.perf_counter() - t0)
    e2e_value = world * e2e_steps / e2e_s

    step_s = ms * 1e-3 / steps
    achieved = DECODE_BYTES / step_s / 1e9
    traffic, traffic_source = profiled_decode_traffic()
    line.update({
        "metric": "int4_moe_layer_tokens_per_s", "value": value, "unit": "tokens/s",
        "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": ms / steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int4 weights, bf16 activations, fp32 accumulate", "data": "synthetic",
        "config": {"workload": "config1_decode_1token_moe_layer", "hidden": D, "experts": E,
                   "top_k": K, "expert_intermediate": F, "shared_intermediate": FS,
                   "layers_rotated": n_layers, "input_rows_rotated": n_rows,
                   "l2_policy": f"weights of {n_layers} layers rotate: "
                                f"{n_layers * DECODE_BYTES / 1e6:.0f} MB touched > 126 MB L2",
                   "multi_gpu": "replicas only (decode does not shard)",
                   "launch": f"one CUDA graph of the {steps} steps, replayed; value = steps / median replay"},
        "timed_region": timing,
        "clocks": clocks,
        "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": D * 2,
                "d2h_bytes_per_step": D * 2, "steps": e2e_steps, "seconds": e2e_s,
                "call": "ff_moe_layer_host, pinned host row in, pinned host row out"},
        "gpu_launches": int(round(steps * kernels_per_step)),
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"],
                     "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"], "traffic": traffic,
                     "traffic_source": traffic_source,
                     "peak_source": peaks["source"], "frac_of_nominal_8TBs": achieved / 8000.0,
                     "kernel": "k_decode_fused: the whole decode step is this one launch",
                     "algorithmic_bytes_per_step": DECODE_BYTES},
        "kernels": kernels,
    })

    # ================= verify: config 2, 16-token blocks =================
    if "verify" in want and rank == 0:
        set_router_bias("normal")
        n_blocks = 16
        vbits = workload.make_tokens(ROOT_SEED, "verify.x", 16 * n_blocks, D)
        vx = hotpath.bf16_tensor(vbits, device)
        vblocks = [vx[16 * i:16 * i + 16].contiguous() for i in range(n_blocks)]
        vy = torch.zeros((16, D), dtype=torch.bfloat16, device=device)

        def verify_step(i):
            ctx.moeLayer(i % n_layers, vblocks[i % n_blocks], vy)

        active = []
        for i in range(n_layers * 2):
            verify_step(i)
            torch.cuda.synchronize()
            active.append(ctx.info().lastActiveExperts)
        vgroup = n_layers * 2
        vms, vtiming, v_per_step, _ = measure_graph(verify_step, vgroup, vgroup, all_ranks=False)
        mean_active = float(np.mean(active))
        vbytes = mean_active * EXPERT_BYTES + SHARED_BYTES + ROUTER_BYTES + 16 * ACT_IO_BYTES
        vach = vbytes / (vms * 1e-3 / vgroup) / 1e9
        hvx = [torch.from_numpy(vbits[16 * i:16 * i + 16].view(np.int16).copy()).view(torch.bfloat16).pin_memory()
               for i in range(n_blocks)]
        hvy = torch.zeros((16, D), dtype=torch.bfloat16).pin_memory()
        for i in range(3):
            ctx.moeLayerHost(i % n_layers, hvx[i % n_blocks], hvy)
        ve2e = 8 if args.quick else 1500
        t0 = time.perf_counter()
        for i in range(ve2e):
            ctx.moeLayerHost(i % n_layers, hvx[i % n_blocks], hvy)
        ve2e_s = time.perf_counter() - t0
        line["verify"] = {
            "workload": "config2_verify_16token_block", "tokens_per_s": 16 * vgroup / (vms * 1e-3),
            "ms_per_step": vms / vgroup, "steps": vgroup, "timed_region": vtiming,
            "active_experts_mean": mean_active, "gpu_launches_per_step": v_per_step,
            "e2e": {"value": 16 * ve2e / ve2e_s, "unit": "tokens/s", "h2d_bytes_per_step": 16 * D * 2,
                    "d2h_bytes_per_step": 16 * D * 2, "steps": ve2e, "seconds": ve2e_s},
            "roofline": {"bound": "hbm", "achieved": vach, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": vach / peaks["hbm_gbs"], "frac_of_nominal_8TBs": vach / 8000.0,
                         "algorithmic_bytes_per_step": vbytes},
            "kernels": {} if args.quick else traced_kernels(ctx, verify_step, vgroup)}

    # ================= prefill: config 3, 4096 tokens, Zipf-skewed routing =================
    if "prefill" in want and rank == 0:
        set_router_bias("zipf")
        pbits = workload.make_tokens(ROOT_SEED, "prefill.x", PREFILL_TOKENS, D)
        px = hotpath.bf16_tensor(pbits, device)
        py = torch.zeros((PREFILL_TOKENS, D), dtype=torch.bfloat16, device=device)
        counter = [0]

        def prefill_step():
            ctx.moeLayer(counter[0] % n_layers, px, py)
            counter[0] += 1

        for _ in range(3):
            prefill_step()
        torch.cuda.synchronize()
        err = ctx.info().deviceErrorFlag
        est = float(np.median(time_replays(torch, torch.cuda.current_stream(), prefill_step, 3)))
        psteps = max(8, int(np.ceil(min_s * 1e3 / max(est, 1e-3))))
        per_step = time_replays(torch, torch.cuda.current_stream(), prefill_step, psteps)
        pms = float(np.median(per_step))
        flops = PREFILL_TOKENS * (2 * (K * 3 * F * D + 3 * FS * D + E * D))
        tf = flops / (pms * 1e-3) / 1e12
        bf16_peak = measured_bf16_peak()
        region_s = float(np.sum(per_step)) * 1e-3
        # a region of under a second runs at burst clocks: the burst cuBLAS figure is its peak
        use_burst = region_s < 1.0
        peak_tf = bf16_peak["burst_tflops"] if use_burst else bf16_peak["tflops"]
        info = ctx.info()
        # flops the GEMM units issue, against the useful ones: a unit is (row tile of up to 192 rows of
        # one expert, rounded up to 32 accumulator columns) x (128 weight rows, 64 gate + 64 up or 128
        # down) x the whole contraction; the pair of weight-row tiles a CTA pair takes is padded to
        # an even count.  From the expert offsets of the last step (read back after the timing).
        _, offsets = hotpath.PrefillGroupedRoutedMoE(ctx).lastRoutes(PREFILL_TOKENS * K)
        counts = np.diff(offsets.astype(np.int64))
        def issued(rows_per_group, f_mid):
            cols = 0
            for c in rows_per_group:
                full, rest = divmod(int(c), 192)
                cols += full * 192 + (max(32, (rest + 31) // 32 * 32) if rest else 0)
            gate_up = 2 * ((-(-f_mid // 64) + 1) // 2) * 128 * D     # weight rows issued x contraction
            down = 2 * ((-(-D // 128) + 1) // 2) * 128 * f_mid
            return 2 * cols * (gate_up + down)
        issued_flops = issued(counts, F) + issued([PREFILL_TOKENS], FS)
        gemm_flops = PREFILL_TOKENS * 2 * (K * 3 * F * D + 3 * FS * D)
        line["prefill"] = {
            "workload": "config3_prefill_4096tokens_zipf", "tokens_per_s": PREFILL_TOKENS / (pms * 1e-3),
            "ms_per_step": pms, "steps": psteps, "timed_region": spread(per_step, 1), "device_error_flag": err,
            "active_experts": info.lastActiveExperts,
            "roofline": {"bound": "tensor", "achieved": tf, "peak": peak_tf, "unit": "TFLOP/s",
                         "frac": tf / peak_tf,
                         "peak_source": ("measured burst" if use_burst else "measured sustained")
                         if bf16_peak["source"].startswith("measured") else "fallback",
                         "frac_of_measured_burst": tf / bf16_peak["burst_tflops"],
                         "frac_of_measured_sustained": tf / bf16_peak["tflops"],
                         "frac_of_nominal_2250TF": tf / 2250.0, "algorithmic_flops_per_step": flops},
            "gemm_flops": {"useful": gemm_flops, "issued": issued_flops, "useful_over_issued": gemm_flops / issued_flops,
                           "row_tiles": int(sum(-(-int(c) // 192) for c in counts)),
                           "note": "issued = accumulator columns (rows of each expert to 32) x weight-row tiles of 128 "
                                   "(an odd tile count padded for the CTA pair) x contraction"},
            "kernels": {} if args.quick else traced_kernels(ctx, lambda i: prefill_step(), 4)}

    # ================= stack: config 4, 30 layers x 32768 tokens, experts sharded over the ranks ====
    if "stack" in want:
        ctx.close()
        ctx = None
        stack = measure_stack(torch, dist, hotpath, workload, host_layers[:min(STACK_DISTINCT_LAYERS, n_layers)],
                              rank, local_rank, world, device, args)
        if rank == 0:
            line["stack"] = stack

    if rank == 0 and world == 1 and not args.quick:
        cpu_rate, cpu_steps, cpu_threads = cpu_decode_baseline(host_layer0, tokens_bits)
        line["cpu_baseline"] = {"value": cpu_rate, "unit": "tokens/s", "cores": cpu_threads,
                                "kind": "port",
                                "sample": f"{cpu_steps} decode steps of the C oracle (OpenMP), one layer",
                                "other_configs": cpu_other_configs(host_layer0, router_bias("normal", 0),
                                                                   router_bias("zipf", 0))}
    if rank == 0:
        emit(line)
    if ctx is not None:
        ctx.close()
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


_RESULT_FD = None


def keep_stdout_for_the_result():
    """Everything libraries print while the bench runs (NCCL's version banner, for one) goes to
    stderr; file descriptor 1 is kept aside for the one JSON line."""
    global _RESULT_FD
    sys.stdout.flush()
    _RESULT_FD = os.dup(1)
    os.dup2(2, 1)


def emit(line: dict):
    text = (json.dumps(line) + "\n").encode()
    if _RESULT_FD is None:
        sys.stdout.write(text.decode())
        sys.stdout.flush()
    else:
        sys.stdout.flush()
        os.write(_RESULT_FD, text)


def run_ep_group(args):
    """`--ep-group`: configuration 4's stack through ff_ep_moe_stack, ONE process driving
    `--gpus` GPUs (run with plain `python`, not torchrun).  The experts of each layer are placed to
    even out the routes a one-device pass over rank 0's rows counted.  Timed by the host clock around
    the synchronous call; the output of rank 0 is compared with ff_moe_stack on one device holding
    every expert.  Prints its own JSON line (not the contract's line)."""
    import time

    import torch
    from ane_fieldfare_b200 import hotpath, parallel, synth, workload
    world = args.gpus
    if torch.cuda.device_count() < world:
        raise SystemExit(f"--ep-group needs {world} GPUs in this process")
    layers = args.stack_layers
    tokens_local = STACK_TOKENS // world
    epr = E // world
    capacity = min(STACK_TOKENS * K, 4 * tokens_local * K)
    host_layers = [workload.make_layer(ROOT_SEED, slot) for slot in range(STACK_DISTINCT_LAYERS)]
    priors = [synth.zipf_log_prior(E, 1.1, ROOT_SEED, f"stack.zipf.{i}") for i in range(len(host_layers))]
    xs = [hotpath.bf16_tensor(workload.make_tokens(ROOT_SEED + r, "stack.x", tokens_local, D), torch.device("cuda", r))
          for r in range(world)]

    # one device, every expert: the expected output of rank 0 and every layer's routes
    full = hotpath.HotpathContext(layers=layers, experts=E, d=D, f=F, sharedF=FS, topK=K, maxTokens=tokens_local,
                                  device=0)
    for slot in range(layers):
        L = host_layers[slot % len(host_layers)]
        full.loadLayer(slot, L.blobs, L.layout.stride, L.layout.offsets)
        full.loadShared(slot, *L.shared_projections())
        full.loadRouter(slot, L.routerW, logitBias=priors[slot % len(host_layers)])
    with torch.cuda.device(0):
        ids = torch.empty((layers, tokens_local, K), dtype=torch.int32, device=xs[0].device)
        want = torch.empty_like(xs[0])
        full.moeStack(0, layers, xs[0], 1e-6, want, ids=ids)
        torch.cuda.synchronize(0)
        counts = [np.bincount(ids[slot].reshape(-1).cpu().numpy(), minlength=E) for slot in range(layers)]
        want = want.cpu()
    full.close()
    placements = [parallel.balanced_placement((counts[slot] + 0.5).tolist(), world) for slot in range(layers)]

    home, expert = [], []
    for r in range(world):
        h = hotpath.HotpathContext(layers=layers, experts=E, d=D, f=F, sharedF=FS, topK=K, maxTokens=tokens_local,
                                   device=r)
        e = hotpath.HotpathContext(layers=layers, experts=epr, d=D, f=F, sharedF=0, topK=1, maxTokens=capacity,
                                   device=r)
        for slot in range(layers):
            L = host_layers[slot % len(host_layers)]
            h.loadShared(slot, *L.shared_projections())
            h.loadRouter(slot, L.routerW, logitBias=priors[slot % len(host_layers)])
            e.loadLayer(slot, np.ascontiguousarray(L.blobs[placements[slot].experts_of(r)]), L.layout.stride,
                        L.layout.offsets, expertCount=epr)
        home.append(h)
        expert.append(e)
    group = hotpath.ExpertParallelGroup(home, expert, capacityRows=capacity)
    for slot in range(layers):
        group.setPlacement(slot, placements[slot].rank_of.numpy(), placements[slot].local_of.numpy())
    ys = [torch.empty_like(x) for x in xs]
    for _ in range(2):
        group.moeStack(0, layers, xs, 1e-6, ys)
    same = bool(torch.equal(ys[0].cpu(), want))
    per = []
    for _ in range(max(3, min(args.steps, 5))):
        t0 = time.perf_counter()
        group.moeStack(0, layers, xs, 1e-6, ys)
        per.append(1e3 * (time.perf_counter() - t0))
    ms = float(np.median(per))
    group.setTracing(True)
    group.moeStack(0, layers, xs, 1e-6, ys)
    group.setTracing(False)
    phases = group.phaseTimes()
    phase_max = {name: round(max(p[name] for p in phases), 3) for name in group.PHASES} if phases else {}
    flags = [int(c.info().deviceErrorFlag) for c in home + expert]
    launches = sum(int(c.info().kernelLaunches) for c in home + expert)
    tf = stack_flops(layers) / (ms * 1e-3) / 1e12
    emit({"metric": "ep_group_stack_tokens_per_s", "value": STACK_TOKENS / (ms * 1e-3), "unit": "tokens/s",
          "n_gpus": world, "processes": 1, "ms_per_stack": ms, "per_call_ms": [round(v, 3) for v in per],
          "timed_by": "host clock around the synchronous ff_ep_moe_stack call", "tflops": tf,
          "config": {"workload": f"config4_stack_{layers}layers_{STACK_TOKENS}tokens", "tokens_per_rank": tokens_local,
                     "experts_per_rank": epr, "capacity_rows": capacity,
                     "placement": "balanced on the routes of rank 0's rows"},
          "phase_ms_per_stack_max_over_ranks": phase_max,
          "phase_note": "CUDA events of one traced call, summed over the layers; copies_home and shared_ffn both start "
                        "at the end of the experts and run side by side",
          "rank0_equals_one_device_stack_bit_for_bit": same, "device_error_flags": flags,
          "kernel_launches_all_contexts": launches, "data": "synthetic"})
    group.close()
    for c in home + expert:
        c.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=4096)
    ap.add_argument("--warmup", type=int, default=64)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=8, help="resident layers the steps rotate over")
    ap.add_argument("--only", default="", help="comma list of decode,verify,prefill,stack (default all)")
    ap.add_argument("--stack-layers", type=int, default=STACK_LAYERS, help="layers of the config-4 stack")
    ap.add_argument("--ep-comm", choices=("nccl", "peer", "both"), default="both",
                    help="how the expert-parallel stack moves rows between ranks (both: time each, report the faster)")
    ap.add_argument("--ep-chunks", type=int, default=2,
                    help="runs the local tokens are cut into per layer under expert parallelism")
    ap.add_argument("--quick", action="store_true",
                    help="skip the end-to-end loop, per-kernel tracing and the CPU baseline (for profiler runs)")
    ap.add_argument("--ep-group", action="store_true",
                    help="time configuration 4's stack through ff_ep_moe_stack: one process driving --gpus GPUs")
    args = ap.parse_args()
    keep_stdout_for_the_result()
    if args.ep_group:
        run_ep_group(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
