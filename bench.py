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
KERNELS_PER_DECODE_STEP = 1
# dram__bytes_read.sum + dram__bytes_write.sum of one decode launch, from an ncu capture of this
# kernel on these shapes (bytes)
NCU_DECODE_TRAFFIC_BYTES = 37_749_760
ROOT_SEED = 0xF1E1DFA2E


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
                 "--format=csv,noheader,nounits", "-lms", "100"],
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
    print(json.dumps(line), flush=True)


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


def capture_steps(torch, ctx, stream, step, group):
    """One CUDA graph holding `group` consecutive steps (a few uncaptured steps run first so that
    every kernel is configured before the capture)."""
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        for i in range(3):
            step(i)
        stream.synchronize()
        with torch.cuda.graph(graph, stream=stream):
            for i in range(group):
                step(i)
    return graph


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


def measure_stack(torch, dist, hotpath, workload, host_layers, rank, local_rank, world, device, args):
    """Benchmark configuration 4: a 30-layer stack of MoE blocks (RMSNorm between layers, no
    attention), 32768 prefill tokens, experts sharded over the ranks with an NCCL all-to-all
    dispatch and combine per layer.  All 30 layer slots are resident (13.2 GB over the box); their
    bytes repeat a few distinct seeded layers, which does not change the work."""
    from ane_fieldfare_b200 import parallel, synth
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29533")
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=device)
    layers = args.stack_layers
    tokens_local = STACK_TOKENS // world
    epr = E // world
    capacity = min(STACK_TOKENS * K, 3 * tokens_local * K)
    home = hotpath.HotpathContext(layers=len(host_layers), experts=E, d=D, f=F, sharedF=FS, topK=K,
                                  maxTokens=tokens_local, device=local_rank)
    local = hotpath.HotpathContext(layers=layers, experts=epr, d=D, f=F, sharedF=0, topK=1,
                                   maxTokens=capacity, device=local_rank)
    placements = []
    for i, L in enumerate(host_layers):
        prior = synth.zipf_log_prior(E, 1.1, ROOT_SEED, f"stack.zipf.{i}")
        home.loadShared(i, *L.shared_projections())
        home.loadRouter(i, L.routerW, logitBias=prior)
        # experts go to ranks so that the expected routed load is balanced (the blob layout is
        # untouched): the load is estimated on the host from the router itself, top-8 over seeded
        # unit-RMS rows, which is what the inter-layer RMSNorm feeds every block
        rows = synth.normal(synth.seedtree_key(ROOT_SEED, f"stack.calib.{i}"), 1024 * D).reshape(1024, D)
        rows /= np.sqrt(np.mean(rows * rows, axis=1, keepdims=True))
        logits = rows.astype(np.float32) @ synth.bf16_to_float(L.routerW).T + prior[None, :]
        chosen = np.argpartition(-logits, K - 1, axis=1)[:, :K]
        load = np.bincount(chosen.reshape(-1), minlength=E).astype(np.float64) + 0.5
        placements.append(parallel.balanced_placement(load, world))
    for slot in range(layers):
        L = host_layers[slot % len(host_layers)]
        mine = placements[slot % len(host_layers)].experts_of(rank)
        local.loadLayer(slot, np.ascontiguousarray(L.blobs[mine]), L.layout.stride, L.layout.offsets,
                        expertCount=epr)
    blocks = []
    for slot in range(layers):
        # the home context is indexed by the distinct layer, the expert context by the stack's slot
        fns = parallel.cuda_layer_fns(home, local, slot % len(host_layers), expert_layer=slot)
        blocks.append(parallel.ExpertParallelMoE(E, K, *fns, placement=placements[slot % len(host_layers)]))
    x0 = hotpath.bf16_tensor(workload.make_tokens(ROOT_SEED + rank, "stack.x", tokens_local, D), device)

    def run_stack():
        x = x0
        for block in blocks:
            x = block.forward(home.rmsnorm(x, None, 1e-6))
        return x

    for _ in range(2):
        run_stack()
    torch.cuda.synchronize()
    dist.barrier()
    steps = 3
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record()
    for _ in range(steps):
        y = run_stack()
    end.record()
    torch.cuda.synchronize()
    ms = begin.elapsed_time(end) / steps
    t = torch.tensor([ms], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    recv = torch.tensor([float(blocks[-1].last_recv_rows)], dtype=torch.float64, device=device)
    rows = [torch.zeros_like(recv) for _ in range(world)]
    dist.all_gather(rows, recv)
    finite = bool(torch.isfinite(y.float()).all().item())
    err = home.info().deviceErrorFlag | local.info().deviceErrorFlag
    flops = layers * STACK_TOKENS * (2 * (K * 3 * F * D + 3 * FS * D + E * D))
    peak = measured_bf16_peak()
    home.close()
    local.close()
    tf = flops / (ms * 1e-3) / 1e12
    return {"workload": f"config4_stack_{layers}layers_{STACK_TOKENS}tokens_expert_parallel", "gpus": world,
            "tokens_per_s": STACK_TOKENS / (ms * 1e-3), "ms_per_stack": ms, "steps": steps,
            "tflops": tf, "frac_of_measured_bf16_per_gpu": tf / (peak["tflops"] * world),
            "last_layer_rows_received_per_rank": [int(r.item()) for r in rows],
            "output_finite": finite, "device_error_flag": int(err),
            "collective": "NCCL all_to_all_single (dispatch + combine per layer)",
            "placement": "experts assigned to ranks by greedy balancing of a load estimated from the router on seeded rows"}


def run_ours(args):
    import torch
    import torch.distributed as dist
    from ane_fieldfare_b200 import hotpath, workload

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

    def set_router_bias(kind):
        from ane_fieldfare_b200 import synth
        for slot in range(n_layers):
            router = host_layers[slot].routerW if slot < STACK_DISTINCT_LAYERS else host_layers[slot][0]
            if kind == "none":
                bias = None
            elif kind == "normal":
                bias = synth.normal(synth.seedtree_key(ROOT_SEED, f"bench.bias.{slot}"), E).astype(np.float32)
            else:
                bias = synth.zipf_log_prior(E, 1.1, ROOT_SEED, f"bench.zipf.{slot}")
            ctx.loadRouter(slot, router, logitBias=bias)

    def sync_max(ms):
        if world > 1:
            t = torch.tensor([ms], dtype=torch.float64, device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item())
        return ms

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
    for i in range(max(args.warmup, 3)):
        decode_step(i)
    torch.cuda.synchronize()
    group = n_layers * 8
    graph = capture_steps(torch, ctx, stream, decode_step, group)
    replays = max(1, (args.steps + group - 1) // group)
    steps = replays * group
    time_graph(torch, stream, graph, max(1, (args.warmup + group - 1) // group))
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ms = time_graph(torch, stream, graph, replays)
    torch.cuda.synchronize()
    clocks = sampler.stop() if rank == 0 else None
    ms = sync_max(ms)
    if world > 1:
        dist.barrier()
    value = world * steps / (ms * 1e-3)
    kernels = {} if args.quick else traced_kernels(ctx, decode_step, group)

    # end to end through the host-buffer entry point
    hx = [torch.from_numpy(tokens_bits[i:i + 1].view(np.int16).copy()).view(torch.bfloat16).pin_memory()
          for i in range(n_rows)]
    hy = torch.zeros((1, D), dtype=torch.bfloat16).pin_memory()
    e2e_steps = 8 if args.quick else min(steps, 2000)
    for i in range(5):
        ctx.moeLayerHost(i % n_layers, hx[i % n_rows], hy)
    if world > 1:
        dist.barrier()
    t0 = time.perf_counter()
    for i in range(e2e_steps):
        ctx.moeLayerHost(i % n_layers, hx[i % n_rows], hy)
    e2e_s = sync_max(time.perf_counter() - t0)
    e2e_value = world * e2e_steps / e2e_s

    step_s = ms * 1e-3 / steps
    achieved = DECODE_BYTES / step_s / 1e9
    line.update({
        "metric": "int4_moe_layer_tokens_per_s", "value": value, "unit": "tokens/s",
        "n_gpus": world, "steps": steps, "warmup": max(args.warmup, 3), "ms_per_step": ms / steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int4 weights, bf16 activations, fp32 accumulate", "data": "synthetic",
        "config": {"workload": "config1_decode_1token_moe_layer", "hidden": D, "experts": E,
                   "top_k": K, "expert_intermediate": F, "shared_intermediate": FS,
                   "layers_rotated": n_layers, "input_rows_rotated": n_rows,
                   "l2_policy": f"weights of {n_layers} layers rotate: "
                                f"{n_layers * DECODE_BYTES / 1e6:.0f} MB touched > 126 MB L2",
                   "multi_gpu": "replicas only (decode does not shard)",
                   "launch": f"CUDA graph of {group} steps"},
        "clocks": clocks,
        "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": D * 2,
                "d2h_bytes_per_step": D * 2, "steps": e2e_steps},
        "gpu_launches": steps * KERNELS_PER_DECODE_STEP,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"],
                     "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"], "traffic": NCU_DECODE_TRAFFIC_BYTES,
                     "peak_source": peaks["source"], "frac_of_nominal_8TBs": achieved / 8000.0,
                     "kernel": "the whole decode step (all kernels of one token through one layer)",
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
        vgraph = capture_steps(torch, ctx, stream, verify_step, vgroup)
        vreplays = max(2, args.steps // (8 * vgroup))
        time_graph(torch, stream, vgraph, 2)
        vms = time_graph(torch, stream, vgraph, vreplays)
        vsteps = vreplays * vgroup
        mean_active = float(np.mean(active))
        vbytes = mean_active * EXPERT_BYTES + SHARED_BYTES + ROUTER_BYTES + 16 * ACT_IO_BYTES
        vach = vbytes / (vms * 1e-3 / vsteps) / 1e9
        line["verify"] = {
            "workload": "config2_verify_16token_block", "tokens_per_s": 16 * vsteps / (vms * 1e-3),
            "ms_per_step": vms / vsteps, "steps": vsteps, "active_experts_mean": mean_active,
            "roofline": {"bound": "hbm", "achieved": vach, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": vach / peaks["hbm_gbs"], "frac_of_nominal_8TBs": vach / 8000.0,
                         "algorithmic_bytes_per_step": vbytes},
            "kernels": traced_kernels(ctx, verify_step, vgroup)}

    # ================= prefill: config 3, 4096 tokens, Zipf-skewed routing =================
    if "prefill" in want and rank == 0:
        set_router_bias("zipf")
        pbits = workload.make_tokens(ROOT_SEED, "prefill.x", PREFILL_TOKENS, D)
        px = hotpath.bf16_tensor(pbits, device)
        py = torch.zeros((PREFILL_TOKENS, D), dtype=torch.bfloat16, device=device)

        def prefill_step(i):
            ctx.moeLayer(i % n_layers, px, py)

        for i in range(3):
            prefill_step(i)
        torch.cuda.synchronize()
        err = ctx.info().deviceErrorFlag
        psteps = max(8, min(64, args.steps // 64))
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        for i in range(psteps):
            prefill_step(i)
        end.record()
        torch.cuda.synchronize()
        pms = begin.elapsed_time(end)
        flops = PREFILL_TOKENS * (2 * (K * 3 * F * D + 3 * FS * D + E * D))
        tf = flops / (pms * 1e-3 / psteps) / 1e12
        bf16_peak = measured_bf16_peak()
        line["prefill"] = {
            "workload": "config3_prefill_4096tokens_zipf", "tokens_per_s": PREFILL_TOKENS * psteps / (pms * 1e-3),
            "ms_per_step": pms / psteps, "steps": psteps, "device_error_flag": err,
            "roofline": {"bound": "tensor", "achieved": tf, "peak": bf16_peak["tflops"], "unit": "TFLOP/s",
                         "frac": tf / bf16_peak["tflops"], "peak_source": bf16_peak["source"],
                         "frac_of_nominal_2250TF": tf / 2250.0, "algorithmic_flops_per_step": flops},
            "kernels": traced_kernels(ctx, prefill_step, 4)}

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
                                "sample": f"{cpu_steps} decode steps of the C oracle (OpenMP), one layer"}
    if rank == 0:
        print(json.dumps(line), flush=True)
    if ctx is not None:
        ctx.close()
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=4096)
    ap.add_argument("--warmup", type=int, default=64)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=8, help="resident layers the steps rotate over")
    ap.add_argument("--only", default="", help="comma list of decode,verify,prefill,stack (default all)")
    ap.add_argument("--stack-layers", type=int, default=STACK_LAYERS, help="layers of the config-4 stack")
    ap.add_argument("--quick", action="store_true",
                    help="skip the end-to-end loop, per-kernel tracing and the CPU baseline (for profiler runs)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
