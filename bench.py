#!/usr/bin/env python
"""Benchmark of the HLQ LUT-GEMV path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W]            # this implementation
    python bench.py --impl reference [--steps K] [--warmup W]      # CPU restatement of the reference

Workload (N = 1 and per rank for N > 1): the Llama-3-8B decoder projection set at w2g128,
batch 1, fp16 activations ~ N(0,1): per layer q/o 4096x4096, k/v 1024x4096, gate/up
14336x4096, down 4096x14336, 32 layers with distinct seeded random weights (bit-planes
Bernoulli(0.5), alpha = |N(0, 0.02)|, z ~ N(0, 0.01)), 2.07 GB of packed weights per step, so
nothing stays in the 126 MB L2 between steps.  One step = one pass over all 224 projections =
the linear work of one decoded token.

Metric: GB/s on ALGORITHMIC bytes (bit-planes + fp16 scales + fp16 zeros as exported:
q/8 + 2(q+1)/g bytes per weight), whole job over all ranks.  With N > 1 every rank streams its
own replica of the set (data-parallel decode, no collective): weak scaling.

One JSON line is printed by rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

NCU_TRAFFIC_RATIO = (130.33 + 3.70) / 129.50   # dram__bytes_read + write over algorithmic bytes
HBM_NOMINAL_GBS = 8000.0
FALLBACK_PEAK_GBS = 6650.0


def projection_set(hidden=4096, ffn=14336, kv=1024, fuse=False):
    """(name, out_channel, in_channel) of one decoder layer."""
    if fuse:
        return [("qkv", hidden + 2 * kv, hidden), ("o", hidden, hidden),
                ("gate_up", 2 * ffn, hidden), ("down", hidden, ffn)]
    return [("q", hidden, hidden), ("k", kv, hidden), ("v", kv, hidden), ("o", hidden, hidden),
            ("gate", ffn, hidden), ("up", ffn, hidden), ("down", hidden, ffn)]


def algorithmic_bytes(n, k, q, g):
    return q * n * k // 8 + 2 * (q + 1) * n * (k // g)


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_PEAK_GBS, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while running."""

    REASONS = {
        0x0000000000000004: "sw_power_cap",
        0x0000000000000008: "hw_slowdown",
        0x0000000000000020: "sw_thermal_slowdown",
        0x0000000000000040: "hw_thermal_slowdown",
    }

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._t = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _poll(self):
        try:
            self.samples.append(self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM))
            mask = self.nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
            for bit, name in self.REASONS.items():
                if mask & bit:
                    self.reasons.add(name)
        except Exception:
            pass

    def start(self):
        if self.nv is None:
            return

        def loop():
            while not self._stop.is_set():
                self._poll()
                time.sleep(0.004)
        self._t = threading.Thread(target=loop, daemon=True)
        self._t.start()

    def stop(self):
        if self.nv is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        self._poll()
        self._stop.set()
        if self._t:
            self._t.join()
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


# ------------------------------------------------------------------------------------------
# CPU arm: the restatement of the reference's NEON kernel on the host cores
# ------------------------------------------------------------------------------------------
def cpu_threads():
    from oracle import cpu_baseline
    avail = min(os.cpu_count() or 1, cpu_baseline.max_threads())
    t = 1
    while t * 2 <= min(avail, 32):     # rows per thread chunk must stay multiples of 32
        t *= 2
    return t


def build_cpu_sample(layers, q, g, threads, seed=0):
    from oracle import cpu_baseline, hlq_oracle as O
    lins, xs, total = [], [], 0
    for layer in range(layers):
        for pi, (_, n, k) in enumerate(projection_set()):
            d = O.synth_linear(n, k, q, g, m=1, seed=seed + layer * 16 + pi)
            lins.append(cpu_baseline.CpuLinear(d["w_quant"], d["w_scale"], d["w_zero"], g, threads=threads))
            xs.append(d["x"])
            total += algorithmic_bytes(n, k, q, g)
    return lins, xs, total


def time_cpu_sample(lins, xs, steps, warmup):
    for _ in range(warmup):
        for lin, x in zip(lins, xs):
            lin.forward(x)
    t0 = time.perf_counter()
    for _ in range(steps):
        for lin, x in zip(lins, xs):
            lin.forward(x)
    return (time.perf_counter() - t0) / steps


def run_reference(args):
    """Reference arm: the reference's CPU LUT kernel (its C restatement: the NEON sources do
    not compile for x86-64) on the host cores, same metric, on a bounded sample."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import build as obuild
    obuild.build()
    threads = cpu_threads()
    layers = args.cpu_layers
    lins, xs, total = build_cpu_sample(layers, args.bits, args.groupsize, threads)
    steps = max(1, min(args.steps, 50))
    sec = time_cpu_sample(lins, xs, steps, min(args.warmup, 3))
    gbs = total / sec / 1e9
    sample = f"{layers} of 32 layers of the projection set ({total} bytes) per step"
    line = {
        "impl": "reference", "metric": "hlq_gemv_gbs", "value": gbs, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": min(args.warmup, 3), "ms_per_step": sec * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16",
        "data": "synthetic",
        "config": workload_config(args, fused=False),
        "decode_tokens_per_s": 1.0 / (sec * 32 / layers),
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(args, fused):
    return {"workload": f"llama3-8b projection set w{args.bits}g{args.groupsize}, batch {args.batch}, "
                        f"{args.layers} layers", "bits": args.bits, "groupsize": args.groupsize,
            "batch": args.batch, "layers": args.layers, "fused_qkv_gate_up": bool(fused),
            "l2": "inputs (2.07 GB of weights per step) larger than L2; no flush needed",
            "launch": ("cuda graph of one step" if not args.no_graph else "stream launches")
                      + {"none": ", one launch per projection", "layer": ", one grouped launch per layer",
                         "model": ", one grouped launch per step"}[args.group]}


# ------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------
def run_gpu(args):
    import torch
    import torch.distributed as dist
    from elutq_b200 import _lib
    from elutq_b200.format import ExportedLinear
    from elutq_b200.linear import HLQWeight, Workspace, workspace_bytes

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback for the GPU arm)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    L = _lib.lib()
    q, g, m = args.bits, args.groupsize, args.batch
    dt = torch.float16

    # ---- weights: distinct seeded random tensors per layer, generated on the device
    gen = torch.Generator(device=dev)
    weights, shapes, total_bytes = [], [], 0
    for layer in range(args.layers):
        for pi, (_, n, k) in enumerate(projection_set(fuse=args.fuse)):
            gen.manual_seed(args.seed + 1000 * rank + layer * 16 + pi)
            wq = torch.randint(0, 256, (q, n, k // 8), dtype=torch.uint8, device=dev, generator=gen)
            ws = (torch.randn((q, n, k // g), device=dev, generator=gen) * 0.02).abs().half()
            wz = (torch.randn((n, k // g), device=dev, generator=gen) * 0.01).half()
            lin = ExportedLinear(wq, ws, wz, None, g)
            weights.append(HLQWeight.from_export(lin, device=local))
            shapes.append((n, k))
            total_bytes += algorithmic_bytes(n, k, q, g)
            del wq, ws, wz, lin
    nlin = len(weights)

    # ---- activations / outputs: one packed buffer each, plus pinned host mirrors
    xoff, yoff = [0], [0]
    for n, k in shapes:
        xoff.append(xoff[-1] + m * k)
        yoff.append(yoff[-1] + m * n)
    gen.manual_seed(args.seed + 7)
    x_all = torch.randn(xoff[-1], device=dev, generator=gen).to(dt)
    y_all = torch.zeros(yoff[-1], dtype=dt, device=dev)
    x_host = x_all.cpu().pin_memory()
    y_host = torch.empty_like(y_all, device="cpu").pin_memory()
    ws_bytes = max(workspace_bytes(m, k, n, q, g) for n, k in shapes)
    ws = Workspace(ws_bytes, dev)
    stream = torch.cuda.Stream(device=dev)

    xs = [x_all[xoff[i]:xoff[i + 1]].view(m, k) for i, (n, k) in enumerate(shapes)]
    ys = [y_all[yoff[i]:yoff[i + 1]].view(m, n) for i, (n, k) in enumerate(shapes)]
    groups = []
    if args.group != "none":
        from elutq_b200.linear import HLQGroup
        per = len(projection_set(fuse=args.fuse)) if args.group == "layer" else nlin
        for a0 in range(0, nlin, per):
            grp = HLQGroup(weights[a0:a0 + per], max_m=m)
            grp.bind(xs[a0:a0 + per], ys[a0:a0 + per])
            groups.append(grp)

    def one_step(sptr):
        if groups:
            for grp in groups:
                st = L.hlq_group_forward(grp.handle, m, sptr)
                if st:
                    _lib.check(st, "hlq_group_forward")
            return
        for i, (n, k) in enumerate(shapes):
            st = L.hlq_linear_forward(m, k, n, x_all.data_ptr() + 2 * xoff[i], _lib.HLQ_F16,
                                      y_all.data_ptr() + 2 * yoff[i], _lib.HLQ_F16, ws.ptr, ws.nbytes,
                                      weights[i].handle, sptr)
            if st:
                _lib.check(st, "hlq_linear_forward")

    torch.cuda.synchronize()
    with torch.cuda.stream(stream):
        before = L.hlq_kernel_launch_count()
        one_step(stream.cuda_stream)          # also configures the kernels before any capture
        launches_per_step = L.hlq_kernel_launch_count() - before
        stream.synchronize()
        assert ws.kernel_status() == 0 and all(g_.kernel_status() == 0 for g_ in groups)
        if args.no_graph:
            def step():
                one_step(stream.cuda_stream)
        else:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                one_step(torch.cuda.current_stream().cuda_stream)

            def step():
                graph.replay()

        def barrier():
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()

        # ---- device-resident timing
        for _ in range(args.warmup):
            step()
        barrier()
        sampler = ClockSampler(local)
        sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(args.steps):
            step()
        e1.record(stream)
        barrier()
        clocks = sampler.stop()
        ms = e0.elapsed_time(e1)

        # ---- end to end: host activations in, host outputs back, every step
        for _ in range(min(args.warmup, 3)):
            x_all.copy_(x_host, non_blocking=True)
            step()
            y_host.copy_(y_all, non_blocking=True)
        barrier()
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        f0.record(stream)
        for _ in range(args.steps):
            x_all.copy_(x_host, non_blocking=True)
            step()
            y_host.copy_(y_all, non_blocking=True)
        f1.record(stream)
        barrier()
        ms_e2e = f0.elapsed_time(f1)
        assert ws.kernel_status() == 0 and all(g_.kernel_status() == 0 for g_ in groups)

    t = torch.tensor([ms, ms_e2e], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, ms_e2e = float(t[0]), float(t[1])
    sec_step = ms / 1e3 / args.steps
    value = world * total_bytes / sec_step / 1e9
    e2e_value = world * total_bytes / (ms_e2e / 1e3 / args.steps) / 1e9
    peak, peak_kind = measured_peak()
    per_gpu = value / world

    # DRAM bytes per launch: one ncu capture of a 2-layer launch of this kernel (w2g128, batch 1)
    # read 130.33 MB and wrote 3.70 MB for 129.50 MB of algorithmic bytes; the traffic grows in
    # proportion to the units a launch processes, so other launches are scaled from that ratio.
    if args.traffic is not None:
        traffic, traffic_source = args.traffic, "--traffic"
    elif args.bits == 2 and args.groupsize == 128 and args.batch == 1:
        traffic = NCU_TRAFFIC_RATIO * total_bytes / max(1, launches_per_step)   # this rank, per launch
        traffic_source = "ncu capture of a 2-layer launch, scaled by algorithmic bytes"
    else:
        traffic, traffic_source = None, "no capture of this configuration"
    line = {
        "metric": "hlq_gemv_gbs", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": sec_step * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32 accumulate over fp16 activations, 1-bit planes",
        "data": "synthetic",
        "config": workload_config(args, args.fuse),
        "pct_of_8tbs_per_gpu": 100.0 * per_gpu / HBM_NOMINAL_GBS,
        "decode_tokens_per_s": world * (32.0 / args.layers) / sec_step,
        "algorithmic_bytes_per_step": total_bytes,
        "clocks": clocks,
        "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": int(x_all.numel() * 2),
                "d2h_bytes_per_step": int(y_all.numel() * 2)},
        "gpu_launches": int(launches_per_step * args.steps),
        "roofline": {"bound": "hbm", "achieved": per_gpu, "peak": peak, "unit": "GB/s",
                     "frac": per_gpu / peak, "traffic": traffic, "traffic_source": traffic_source,
                     "peak_source": f"of {peak_kind}", "kernel": "lut8_gemv_kernel",
                     "launches_per_step": int(launches_per_step),
                     "avg_launch_us": sec_step * 1e6 / max(1, launches_per_step)},
    }
    if world > 1:
        dist.barrier()
    if rank == 0:
        if world == 1 and not args.skip_cpu:
            from oracle import build as obuild
            obuild.build()
            threads = cpu_threads()
            lins, xs, cpu_total = build_cpu_sample(args.cpu_layers, q, g, threads)
            sec = time_cpu_sample(lins, xs, args.cpu_steps, 1)
            line["cpu_baseline"] = {
                "value": cpu_total / sec / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
                "sample": f"{args.cpu_layers} of 32 layers of the projection set ({cpu_total} bytes), "
                          f"{args.cpu_steps} passes"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_decode(args):
    """Whole-token decode of a random-init Llama-shaped decoder, tensor-parallel over the
    ranks (--workload decode).  Reports tokens/s; the linears' algorithmic bytes per token
    over the step time is given beside it."""
    import torch
    import torch.distributed as dist
    from elutq_b200.decoder import PRESETS, TPDecoder
    import dataclasses

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    cfg = PRESETS[args.model]
    if args.decode_layers:
        cfg = dataclasses.replace(cfg, layers=args.decode_layers)
    cfg = dataclasses.replace(cfg, bits=args.bits, groupsize=args.groupsize)
    dec = TPDecoder(cfg, dev, rank, world, seed=args.seed, grouped=not args.ungrouped,
                    fused_allreduce=args.fused_allreduce, fused_glue=not args.torch_glue)
    if args.no_graph:
        # eager steps (for a profiler's launch list; the numbers then include host launch gaps)
        class _Eager:
            def replay(self):
                dec.step_eager(None)
        for _ in range(2):
            dec.step_eager(1)
        graph = _Eager()
    else:
        graph = dec.capture(1)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
    for _ in range(args.warmup):
        graph.replay()
    barrier()
    sampler = ClockSampler(local)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        graph.replay()
    e1.record()
    barrier()
    clocks = sampler.stop()
    t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
    lb = torch.tensor([float(dec.linear_bytes)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(lb, op=dist.ReduceOp.SUM)
    sec = float(t[0]) / 1e3 / args.steps
    # end to end: the token id comes from pinned host memory and the next token goes back to it
    tok_in = torch.ones(1, dtype=torch.int64).pin_memory()
    tok_out = torch.zeros(1, dtype=torch.int64).pin_memory()
    barrier()
    e0.record()
    for _ in range(args.steps):
        dec.token.copy_(tok_in, non_blocking=True)
        graph.replay()
        tok_out.copy_(dec.next_token, non_blocking=True)
        torch.cuda.current_stream().synchronize()
    e1.record()
    barrier()
    t2 = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t2, op=dist.ReduceOp.MAX)
    sec_e2e = float(t2[0]) / 1e3 / args.steps
    if rank == 0:
        print(json.dumps({
            "metric": "decode_tokens_per_s", "value": 1.0 / sec, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": f"{args.model} decode, batch 1, context {cfg.ctx}, w{cfg.bits}g{cfg.groupsize}, "
                                   f"{cfg.layers} layers, tensor-parallel x{world}",
                       "glue": ("PyTorch ops (norm, rope, attention, silu, lm_head) inside one CUDA graph"
                                if args.torch_glue else
                                "own kernels (residual+RMSNorm, RoPE+KV append+attention, gated SiLU, argmax), "
                                "w4g128 HLQ lm_head, " + ("eager launches" if args.no_graph else "one CUDA graph")),
                       "collectives": ("all-reduce fused into the o and down GEMV kernels (peer stores over NVLink)"
                                       if args.fused_allreduce else "NCCL all-reduce after o and down")
                                      + ", NCCL all-gather of the arg-max"},
            "e2e": {"value": 1.0 / sec_e2e, "unit": "tokens/s", "h2d_bytes_per_step": 8, "d2h_bytes_per_step": 8},
            "gpu_launches": int(dec.launches_per_step() * args.steps),
            "linear_algorithmic_bytes_per_token": float(lb[0]),
            "linear_gbs_over_step_time": float(lb[0]) / sec / 1e9,
            "clocks": clocks}), flush=True)
    if world > 1:
        # a communicator cannot be torn down while a captured graph still holds its kernels
        dist.barrier()
        torch.cuda.synchronize()
        dec.graph = None
        del graph
        import gc
        gc.collect()
        torch.cuda.synchronize()
        sys.stdout.flush()
        os._exit(0)


def run_prefill(args):
    """Prefill GEMM (--workload prefill): the Llama-2-13B projection set (hidden 5120, ffn 13824)
    at w2g64 with --tokens bf16 tokens through the dequantize + tcgen05 path.  Reports
    TFLOP/s (2*m*n*k per projection) over --layers layers of distinct random weights."""
    import torch
    from elutq_b200 import _lib
    from elutq_b200.format import ExportedLinear
    from elutq_b200.linear import HLQWeight, Workspace, workspace_bytes, linear_forward

    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    q, g, m = args.bits, 64, args.tokens
    hidden, ffn = 5120, 13824
    shapes = [(hidden, hidden)] * 4 + [(ffn, hidden)] * 2 + [(hidden, ffn)]
    gen = torch.Generator(device=dev)
    weights, flops = [], 0.0
    for layer in range(args.layers):
        for pi, (n, k) in enumerate(shapes):
            gen.manual_seed(args.seed + layer * 16 + pi)
            wq = torch.randint(0, 256, (q, n, k // 8), dtype=torch.uint8, device=dev, generator=gen)
            ws = (torch.randn((q, n, k // g), device=dev, generator=gen) * 0.02).abs().half()
            wz = (torch.randn((n, k // g), device=dev, generator=gen) * 0.01).half()
            weights.append((HLQWeight.from_export(ExportedLinear(wq, ws, wz, None, g), device=local), n, k))
            flops += 2.0 * m * n * k
    xs = {k: torch.randn((m, k), device=dev, generator=gen).bfloat16() for k in (hidden, ffn)}
    ys = {n: torch.empty((m, n), dtype=torch.bfloat16, device=dev) for n in (hidden, ffn)}
    ws_ = Workspace(max(workspace_bytes(m, k, n, q, g) for _, n, k in weights), dev)
    L = _lib.lib()
    before = L.hlq_kernel_launch_count()

    def step():
        for w, n, k in weights:
            linear_forward(xs[k], w, ws_, out=ys[n], impl=_lib.IMPL_GEMM)
    step()
    launches = L.hlq_kernel_launch_count() - before
    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    sampler = ClockSampler(local)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    assert ws_.kernel_status() == 0
    sec = e0.elapsed_time(e1) / 1e3 / args.steps
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            pk = json.load(f)
        peak, kind = float(pk["bf16_tflops_sustained"]), "measured, sustained"
    except Exception:
        peak, kind = 1400.0, "fallback"
    tf = flops / sec / 1e12
    print(json.dumps({
        "metric": "hlq_prefill_tflops", "value": tf, "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "fp16 operands (weights dequantized to fp16, bf16 tokens converted), f32 accumulate",
        "data": "synthetic",
        "config": {"workload": f"llama2-13b projection set w{q}g{g}, {m} bf16 tokens, {args.layers} layers"},
        "gpu_launches": int(launches * args.steps), "clocks": clocks,
        "roofline": {"bound": "tensor", "achieved": tf, "peak": peak, "unit": "TFLOP/s", "frac": tf / peak,
                     "traffic": None, "peak_source": f"of {kind}", "kernel": "dequant_gemm_kernel"}}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--bits", type=int, default=2)
    ap.add_argument("--groupsize", type=int, default=128)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--fuse", action="store_true", help="load q/k/v and gate/up as one weight each")
    ap.add_argument("--no-graph", action="store_true", help="launch from the host every step")
    ap.add_argument("--group", default="model", choices=["none", "layer", "model"],
                    help="run the projections as one persistent launch per layer / per step, "
                         "or as one launch per projection")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--cpu-layers", type=int, default=4)
    ap.add_argument("--cpu-steps", type=int, default=10)
    ap.add_argument("--skip-cpu", action="store_true")
    ap.add_argument("--traffic", type=float, default=None,
                    help="DRAM bytes per launch from an ncu capture, copied into the roofline object")
    ap.add_argument("--workload", default="gemv", choices=["gemv", "decode", "prefill"])
    ap.add_argument("--tokens", type=int, default=2048, help="prefill: rows of activations")
    ap.add_argument("--model", default="llama3-70b", help="decoder preset of --workload decode")
    ap.add_argument("--decode-layers", type=int, default=0, help="override the preset's layer count")
    ap.add_argument("--ungrouped", action="store_true", help="decode: one launch per projection")
    ap.add_argument("--torch-glue", action="store_true", help="decode: PyTorch ops between the linears")
    ap.add_argument("--fused-allreduce", action="store_true",
                    help="decode: sum the row-parallel outputs inside the GEMV kernel instead of NCCL")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "decode":
        run_decode(args)
    elif args.workload == "prefill":
        run_prefill(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
