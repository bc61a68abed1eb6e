#!/usr/bin/env python
"""Benchmark of the HLQ hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W]            # this implementation
    python bench.py --impl reference [--steps K] [--warmup W]      # CPU restatement of the reference

Default workload (every N): ONE random-init Llama-3-70B-shaped decoder (hidden 8192, ffn 28672,
80 layers, 64 q / 8 kv heads of 128, vocabulary 128256; w2g128 HLQ linears, w4g128 lm_head as
the reference exports it), batch 1, context 2048, sharded over the N ranks: q/k/v/gate/up and
lm_head column-parallel, o/down row-parallel with the all-reduce fused into the GEMV kernel.
One step = one decoded token.  The metric is tokens/s of the whole job (strong scaling: the
model is fixed, the ranks share it).  Weights (20.9 GB) are far larger than L2, so no flush is
needed between steps.

At N = 1 the line also carries the other configurations of the path, each measured on the
same GPU in the same run:
  gemv     the Llama-3-8B projection set at w2g128, batch 1 (GB/s on algorithmic bytes)
  batches  the same set at w3g128 with 1, 4, 8 and 16 rows of activations
  prefill  the Llama-2-13B projection set at w2g64 with 2048 bf16 tokens (TFLOP/s)
  cpu_baseline  the C restatement of the reference's CPU kernel on the host cores

`--workload gemv|prefill` run one of those alone.  One JSON line is printed by rank 0.
"""
from __future__ import annotations

import argparse
import dataclasses
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

NCU_TRAFFIC_RATIO = (130.33 + 3.70) / 129.50   # dram__bytes_read + write over algorithmic bytes (lut8_gemv_kernel)
NCU_TRAFFIC_RATIO_CHAIN = (294.63 + 6.50) / 292.6   # the same for decode_chain_kernel (weights + KV cache of a 4-layer capture)
HBM_NOMINAL_GBS = 8000.0
FALLBACK_PEAK_GBS = 6650.0
REPEATS = 5                                    # timed blocks of --steps steps; the median is reported
NORMWISE = "max|y - y_ref| / max|y_ref| (normwise), gate 1e-3 for 16-bit outputs, 1e-5 for fp32"


def projection_set(hidden=4096, ffn=14336, kv=1024):
    """(name, out_channel, in_channel) of one decoder layer."""
    return [("q", hidden, hidden), ("k", kv, hidden), ("v", kv, hidden), ("o", hidden, hidden),
            ("gate", ffn, hidden), ("up", ffn, hidden), ("down", hidden, ffn)]


def algorithmic_bytes(n, k, q, g):
    return q * n * k // 8 + 2 * (q + 1) * n * (k // g)


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            pk = json.load(f)
        return {"hbm": float(pk["hbm_gbs"]), "tf_sustained": float(pk["bf16_tflops_sustained"]),
                "tf_burst": float(pk["bf16_tflops"]), "kind": "measured"}
    except Exception:
        return {"hbm": FALLBACK_PEAK_GBS, "tf_sustained": 1400.0, "tf_burst": 1590.0, "kind": "fallback"}


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


def timed_blocks(step, steps, barrier, stream, device_index, repeats=REPEATS):
    """`repeats` blocks of exactly `steps` steps, each bracketed by a barrier and a device
    synchronize and timed with CUDA events on the launching stream.  Returns the per-block
    milliseconds and the clock record of every block."""
    import torch
    ms, clocks = [], []
    for _ in range(repeats):
        barrier()
        sampler = ClockSampler(device_index)
        sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(steps):
            step()
        e1.record(stream)
        barrier()
        clocks.append(sampler.stop())
        ms.append(e0.elapsed_time(e1))
    return ms, clocks


def merge_clocks(clocks):
    mhz = [c["sm_mhz"] for c in clocks if c.get("sm_mhz") is not None]
    reasons = sorted({r for c in clocks for r in c.get("reasons", [])})
    return {"sm_mhz": statistics.median(mhz) if mhz else None,
            "sm_max_mhz": next((c["sm_max_mhz"] for c in clocks if c.get("sm_max_mhz")), None),
            "reasons": reasons, "samples": sum(c.get("samples", 0) for c in clocks),
            "sm_mhz_per_repeat": mhz}


# ------------------------------------------------------------------------------------------
# CPU arm: the restatement of the reference's NEON kernel on the host cores
# ------------------------------------------------------------------------------------------
def host_cores():
    """Cores this process may run on.  Not omp_get_max_threads(): a launcher that exports
    OMP_NUM_THREADS=1 would turn the CPU arm into a single thread."""
    try:
        return len(os.sched_getaffinity(0))
    except Exception:
        return os.cpu_count() or 1


def cpu_model():
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("model name"):
                    return line.split(":", 1)[1].strip()
    except Exception:
        pass
    return "unknown"


def threads_for(n, cores, cap=64):
    """Largest thread count <= cores that the reference's row split accepts for n output rows:
    ceil(n / threads) must be a multiple of 32 (arm_t_mac_kernal.cpp:483-489)."""
    for t in range(min(cores, cap), 0, -1):
        chunk = (n + t - 1) // t
        if chunk % 32 == 0 and chunk * (t - 1) < n:
            return t
    return 1


class CpuDecodeSample:
    """The linears of `layers` decoder layers of the 70B shape plus the w4g128 lm_head, loaded
    the way the reference's load_Parameter does, for the C restatement of its kernel."""

    def __init__(self, cfg, layers, cores, seed=0):
        from oracle import cpu_baseline, hlq_oracle as O
        self.cfg, self.layers, self.cores = cfg, layers, cores
        q_dim, kv_dim = cfg.n_heads * cfg.head_dim, cfg.n_kv * cfg.head_dim
        shapes = [(q_dim, cfg.hidden), (kv_dim, cfg.hidden), (kv_dim, cfg.hidden), (cfg.hidden, q_dim),
                  (cfg.ffn, cfg.hidden), (cfg.ffn, cfg.hidden), (cfg.hidden, cfg.ffn)]
        self.body, self.body_bytes, self.threads_used = [], 0, set()
        for layer in range(layers):
            for pi, (n, k) in enumerate(shapes):
                d = O.synth_linear(n, k, cfg.bits, cfg.groupsize, m=1, seed=seed + layer * 16 + pi)
                t = threads_for(n, cores)
                self.threads_used.add(t)
                self.body.append((cpu_baseline.CpuLinear(d["w_quant"], d["w_scale"], d["w_zero"], cfg.groupsize,
                                                         threads=t), d["x"]))
                self.body_bytes += algorithmic_bytes(n, k, cfg.bits, cfg.groupsize)
        d = O.synth_linear(cfg.vocab, cfg.hidden, 4, 128, m=1, seed=seed + 100007)
        t = threads_for(cfg.vocab, cores)
        self.threads_used.add(t)
        self.head = (cpu_baseline.CpuLinear(d["w_quant"], d["w_scale"], d["w_zero"], 128, threads=t), d["x"])
        self.head_bytes = algorithmic_bytes(cfg.vocab, cfg.hidden, 4, 128)

    def step(self):
        t0 = time.perf_counter()
        for lin, x in self.body:
            lin.forward(x)
        t1 = time.perf_counter()
        self.head[0].forward(self.head[1])
        return t1 - t0, time.perf_counter() - t1

    def run(self, steps, warmup):
        for _ in range(warmup):
            self.step()
        body = head = 0.0
        for _ in range(steps):
            b, h = self.step()
            body += b
            head += h
        body, head = body / steps, head / steps
        token_s = body * self.cfg.layers / self.layers + head      # all layers + lm_head
        return {"tokens_per_s": 1.0 / token_s, "ms_per_token": token_s * 1e3,
                "sample_ms_per_step": (body + head) * 1e3,
                "gbs": (self.body_bytes + self.head_bytes) / (body + head) / 1e9}

    def describe(self):
        return (f"{self.layers} of {self.cfg.layers} layers' linears (unsharded 70B shapes, w{self.cfg.bits}"
                f"g{self.cfg.groupsize}) + the w4g128 lm_head per step, scaled to {self.cfg.layers} layers; linears "
                f"only (the reference's norm/rope/attention ops are not restated in C and not timed, so this is an "
                f"upper bound of its tokens/s); threads per linear {sorted(self.threads_used)} "
                f"(rows per thread must be multiples of 32)")


def cpu_config1(cores):
    """BASELINE config 1: one 4096x4096 w2g128 GEMV, 4 threads (the reference's default,
    main.cpp:41) and all cores; 5 warm-ups + 50 timed iterations each."""
    from oracle import cpu_baseline, hlq_oracle as O
    d = O.synth_linear(4096, 4096, 2, 128, m=1, seed=0)
    out = {"shape": "4096x4096 w2g128, batch 1", "bytes": algorithmic_bytes(4096, 4096, 2, 128)}
    for label, t in (("threads_4", 4), ("all_cores", threads_for(4096, cores))):
        lin = cpu_baseline.CpuLinear(d["w_quant"], d["w_scale"], d["w_zero"], 128, threads=t)
        sec = lin.time_forward(d["x"], iters=50, warmup=5)
        out[label] = {"threads": t, "us": sec * 1e6, "gbs": out["bytes"] / sec / 1e9}
    return out


def decode_config(model, cfg, world, kind):
    return {"workload": f"{model} decode, batch 1, context {cfg.ctx}, w{cfg.bits}g{cfg.groupsize} linears + w4g128 "
                        f"lm_head, {cfg.layers} layers, tensor-parallel x{world}",
            "model": model, "bits": cfg.bits, "groupsize": cfg.groupsize, "layers": cfg.layers, "context": cfg.ctx,
            "parallelism": f"tp{world}",
            "l2": "weights per step (20.9 GB / N per GPU) larger than L2; no flush needed",
            "path": kind}


DECODE_PATH = ("own kernels only: all layers of a token in ONE persistent kernel (decode chain: per layer the stages "
               "q|k|v LUT GEMV, RoPE + KV append + attention, o, gate/up, down; RMSNorm in the table build, residual "
               "adds and gated SiLU in the completion pass, the rank sums of o and down inside the kernel by peer "
               "stores over NVLink at N > 1), then final norm, w4g128 lm_head, argmax; one CUDA graph per step; "
               "NCCL only for the all-gather of the arg-max")
PER_OP_PATH = ("own kernels only, one launch per op (8 per layer): residual+RMSNorm, q/k/v and gate/up as grouped LUT "
               "GEMVs, RoPE + KV append + attention in one kernel, gated SiLU, o/down LUT GEMVs with the all-reduce "
               "fused into the kernel at N > 1, w4g128 lm_head, argmax; one CUDA graph per step")


def run_reference(args):
    """Reference arm: the reference's CPU LUT kernel (its C restatement: the NEON sources do
    not compile for x86-64) on all host cores, same metric and config, on a bounded sample.
    Under a multi-rank launcher rank 0 alone runs it."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import build as obuild
    obuild.build()
    from elutq_b200.decoder import PRESETS
    cfg = dataclasses.replace(PRESETS[args.model], bits=args.bits, groupsize=args.groupsize)
    if args.decode_layers:
        cfg = dataclasses.replace(cfg, layers=args.decode_layers)
    cores = host_cores()
    sample = CpuDecodeSample(cfg, min(args.cpu_layers, cfg.layers), cores, seed=args.seed)
    steps = max(1, args.steps)
    r = sample.run(steps, args.warmup)
    base = {"value": r["tokens_per_s"], "unit": "tokens/s", "cores": max(sample.threads_used), "kind": "port",
            "sample": sample.describe(), "host_cores": cores, "cpu_model": cpu_model(),
            "linear_gbs": r["gbs"]}
    line = {
        "impl": "reference", "metric": "decode_tokens_per_s", "value": r["tokens_per_s"], "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": args.warmup,
        # a timed step is the SAMPLE (the stated layers + lm_head); `value` scales it to the whole model
        "ms_per_step": r["sample_ms_per_step"], "ms_per_token": r["ms_per_token"],
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f16 (the reference's kernel accumulates in fp16)", "data": "synthetic",
        "config": decode_config(args.model, cfg, args.gpus, DECODE_PATH),
        "cpu_baseline": base,
        "e2e": {"value": r["tokens_per_s"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------
# GPU arm: the projection set (configs 2 and 3)
# ------------------------------------------------------------------------------------------
class ProjectionSet:
    """The Llama-3-8B projection set with distinct seeded random weights per layer, on one GPU."""

    def __init__(self, dev, bits, groupsize, layers, seed, max_m):
        import torch
        from elutq_b200.format import ExportedLinear
        from elutq_b200.linear import HLQWeight
        self.dev, self.q, self.g, self.layers, self.max_m = dev, bits, groupsize, layers, max_m
        gen = torch.Generator(device=dev)
        self.weights, self.shapes, self.total_bytes = [], [], 0
        for layer in range(layers):
            for pi, (_, n, k) in enumerate(projection_set()):
                gen.manual_seed(seed + layer * 16 + pi)
                wq = torch.randint(0, 256, (bits, n, k // 8), dtype=torch.uint8, device=dev, generator=gen)
                ws = (torch.randn((bits, n, k // groupsize), device=dev, generator=gen) * 0.02).abs().half()
                wz = (torch.randn((n, k // groupsize), device=dev, generator=gen) * 0.01).half()
                self.weights.append(HLQWeight.from_export(ExportedLinear(wq, ws, wz, None, groupsize),
                                                          device=dev.index))
                self.shapes.append((n, k))
                self.total_bytes += algorithmic_bytes(n, k, bits, groupsize)
                del wq, ws, wz
        m = max_m
        self.xoff, self.yoff = [0], [0]
        for n, k in self.shapes:
            self.xoff.append(self.xoff[-1] + m * k)
            self.yoff.append(self.yoff[-1] + m * n)
        gen.manual_seed(seed + 7)
        self.x_all = torch.randn(self.xoff[-1], device=dev, generator=gen).half()
        self.y_all = torch.zeros(self.yoff[-1], dtype=torch.float16, device=dev)

    def views(self, m):
        """x and y of every projection for m rows (row-major [m, k] / [m, n] inside each slab)."""
        xs = [self.x_all[self.xoff[i]:self.xoff[i] + m * k].view(m, k) for i, (n, k) in enumerate(self.shapes)]
        ys = [self.y_all[self.yoff[i]:self.yoff[i] + m * n].view(m, n) for i, (n, k) in enumerate(self.shapes)]
        return xs, ys

    def measure(self, m, grouping, steps, warmup, stream, repeats=REPEATS, e2e=False, check=True):
        """GB/s on algorithmic bytes for one grouping of the launches:
        'model'  all projections of all layers in ONE persistent launch (their inputs are made
                 independent: an upper bound that no decode step can reach, since o needs q/k/v and
                 down needs gate/up);
        'layer4' the dependency-respecting order of a decode step: per layer one grouped launch for
                 q/k/v, one for o, one grouped launch for gate/up, one for down;
        'none'   one launch per projection."""
        import torch
        from elutq_b200 import _lib
        from elutq_b200.linear import HLQGroup, Workspace, workspace_bytes, linear_forward
        L = _lib.lib()
        xs, ys = self.views(m)
        nlin = len(self.weights)
        per_layer = len(projection_set())
        if grouping == "model":
            parts = [list(range(nlin))]
        elif grouping == "layer4":
            parts = []
            for a0 in range(0, nlin, per_layer):
                parts += [[a0, a0 + 1, a0 + 2], [a0 + 3], [a0 + 4, a0 + 5], [a0 + 6]]
        else:
            parts = [[i] for i in range(nlin)]
        groups = []
        for idx in parts:
            grp = HLQGroup([self.weights[i] for i in idx], max_m=m)
            grp.bind([xs[i] for i in idx], [ys[i] for i in idx])
            groups.append(grp)

        def one_step(sptr):
            for grp in groups:
                st = L.hlq_group_forward(grp.handle, m, sptr)
                if st:
                    _lib.check(st, "hlq_group_forward")
        torch.cuda.synchronize()
        with torch.cuda.stream(stream):
            before = L.hlq_kernel_launch_count()
            one_step(stream.cuda_stream)          # also configures the kernels before any capture
            launches = L.hlq_kernel_launch_count() - before
            stream.synchronize()
            assert all(g_.kernel_status() == 0 for g_ in groups)
            err = None
            if check:
                # one projection of the timed launches against a launch of its own
                i = 3 if nlin > 3 else 0
                n, k = self.shapes[i]
                ws = Workspace(workspace_bytes(m, k, n, self.q, self.g), self.dev)
                y32 = linear_forward(xs[i], self.weights[i], ws, out_dtype=torch.float32)
                stream.synchronize()
                err = float((ys[i].float() - y32).abs().max() / y32.abs().max())
                assert err <= 1e-3, f"grouped launch disagrees with a single launch: {err}"
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                one_step(torch.cuda.current_stream().cuda_stream)
            for _ in range(warmup):
                graph.replay()
            ms, clocks = timed_blocks(graph.replay, steps, torch.cuda.synchronize, stream, self.dev.index, repeats)
            out = {"grouping": grouping, "rows": m, "launches_per_step": int(launches), "steps": steps,
                   "repeats": repeats, "check_vs_single_launch": err}
            sec = statistics.median(ms) / 1e3 / steps
            out.update(ms_per_step=sec * 1e3, gbs=self.total_bytes / sec / 1e9,
                       gbs_min=self.total_bytes / (max(ms) / 1e3 / steps) / 1e9,
                       gbs_max=self.total_bytes / (min(ms) / 1e3 / steps) / 1e9,
                       clocks=merge_clocks(clocks))
            if e2e:
                x_host = self.x_all.cpu().pin_memory()
                y_host = torch.empty_like(self.y_all, device="cpu").pin_memory()

                def e2e_step():
                    self.x_all.copy_(x_host, non_blocking=True)
                    graph.replay()
                    y_host.copy_(self.y_all, non_blocking=True)
                for _ in range(3):
                    e2e_step()
                ms2, _ = timed_blocks(e2e_step, steps, torch.cuda.synchronize, stream, self.dev.index, 3)
                sec2 = statistics.median(ms2) / 1e3 / steps
                out["e2e"] = {"value": self.total_bytes / sec2 / 1e9, "unit": "GB/s",
                              "h2d_bytes_per_step": int(self.x_all.numel() * 2),
                              "d2h_bytes_per_step": int(self.y_all.numel() * 2)}
            assert all(g_.kernel_status() == 0 for g_ in groups)
            del graph
        for grp in groups:
            grp.free()
        return out


def gemv_object(dev, args, stream, steps, warmup, e2e=False):
    """Config 2: the 8B projection set at w2g128, batch 1."""
    peaks = measured_peaks()
    ps = ProjectionSet(dev, 2, 128, args.layers, args.seed, max_m=1)
    top = ps.measure(1, "model", steps, warmup, stream, e2e=e2e)
    dep = ps.measure(1, "layer4", max(5, steps // 2), warmup, stream, repeats=3)
    obj = {"workload": f"llama3-8b projection set w2g128, batch 1, {args.layers} layers",
           "value": top["gbs"], "unit": "GB/s", "min": top["gbs_min"], "max": top["gbs_max"],
           "ms_per_step": top["ms_per_step"], "steps": steps, "repeats": top["repeats"],
           "pct_of_8tbs": 100.0 * top["gbs"] / HBM_NOMINAL_GBS,
           "frac_of_measured_peak": top["gbs"] / peaks["hbm"],
           "algorithmic_bytes_per_step": ps.total_bytes,
           "launch_shape": "all 224 projections in ONE persistent launch with independent inputs: an upper bound, "
                           "not a decode step (o needs q/k/v, down needs gate/up)",
           "dependent_order": {"value": dep["gbs"], "unit": "GB/s", "ms_per_step": dep["ms_per_step"],
                               "launches_per_step": dep["launches_per_step"],
                               "launch_shape": "per layer: q/k/v group, o, gate/up group, down (what a decode step "
                                               "can issue)"},
           "check_vs_single_launch": top["check_vs_single_launch"], "error_measure": NORMWISE,
           "clocks": top["clocks"]}
    if e2e:
        obj["e2e"] = top["e2e"]
    del ps
    return obj, top


def batches_object(dev, args, stream, steps, warmup):
    """Config 3: the same set at w3g128 with 1, 4, 8 and 16 rows of activations; then once more with the
    optional copy of the planes as 4-bit code words (half a byte per weight of extra device memory)."""
    peaks = measured_peaks()
    ps = ProjectionSet(dev, 3, 128, args.layers, args.seed, max_m=16)

    def rows_of(ms):
        rows = {}
        for m in ms:
            r = ps.measure(m, "model", max(3, steps // 4) if m > 1 else steps, 3, stream, repeats=3, check=(m == 1))
            rows[str(m)] = {"ms_per_step": r["ms_per_step"], "gbs": r["gbs"],
                            "frac_of_measured_peak": r["gbs"] / peaks["hbm"], "launches_per_step": r["launches_per_step"]}
        return rows
    out = {"workload": f"llama3-8b projection set w3g128, {args.layers} layers, rows of activations 1/4/8/16",
           "algorithmic_bytes_per_step": ps.total_bytes, "rows": rows_of((1, 4, 8, 16)),
           "note": "bytes do not grow with the rows; 1 row: LUT kernel; 4, 8, 16 rows: one pass over the weights, "
                   "register dequantization + mma.sync (batch_mma_kernel), bound by the integer pipe"}
    extra = 0
    for w in ps.weights:
        before = w.info.device_bytes
        w.build_batch_codes()
        extra += w.info.device_bytes - before
    out["rows_with_code_words"] = rows_of((4, 8, 16))
    out["code_words"] = {"extra_device_bytes": int(extra),
                         "bytes_read_per_step": int(ps.total_bytes + extra // 4),
                         "note": "hlq_weight_build_batch_codes: the kernel reads 4-bit code words instead of the "
                                 "three planes (traffic 1.29x the algorithmic bytes) and skips the bit gathering"}
    del ps
    return out


def prefill_object(dev, args, layers, steps, warmup):
    """Config 4: Llama-2-13B projection set at w2g64, 2048 bf16 tokens, dequantize + tcgen05 GEMM."""
    import torch
    from elutq_b200 import _lib
    from elutq_b200.format import ExportedLinear
    from elutq_b200.linear import HLQWeight, Workspace, workspace_bytes, linear_forward
    peaks = measured_peaks()
    q, g, m = 2, 64, args.tokens
    hidden, ffn = 5120, 13824
    shapes = [(hidden, hidden)] * 4 + [(ffn, hidden)] * 2 + [(hidden, ffn)]
    gen = torch.Generator(device=dev)
    weights, flops = [], 0.0
    for layer in range(layers):
        for pi, (n, k) in enumerate(shapes):
            gen.manual_seed(args.seed + layer * 16 + pi)
            wq = torch.randint(0, 256, (q, n, k // 8), dtype=torch.uint8, device=dev, generator=gen)
            ws = (torch.randn((q, n, k // g), device=dev, generator=gen) * 0.02).abs().half()
            wz = (torch.randn((n, k // g), device=dev, generator=gen) * 0.01).half()
            weights.append((HLQWeight.from_export(ExportedLinear(wq, ws, wz, None, g), device=dev.index), n, k))
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
    for _ in range(warmup):
        step()
    ms, clocks = timed_blocks(step, steps, torch.cuda.synchronize, torch.cuda.current_stream(dev), dev.index, 3)
    assert ws_.kernel_status() == 0
    sec = statistics.median(ms) / 1e3 / steps
    tf = flops / sec / 1e12
    return {"workload": f"llama2-13b projection set w{q}g{g}, {m} bf16 tokens, {layers} layers",
            "value": tf, "unit": "TFLOP/s", "ms_per_step": sec * 1e3, "steps": steps,
            "frac_of_sustained_bf16": tf / peaks["tf_sustained"], "frac_of_burst_bf16": tf / peaks["tf_burst"],
            "peaks": {"sustained": peaks["tf_sustained"], "burst": peaks["tf_burst"], "source": peaks["kind"]},
            "launches_per_step": int(launches), "kernel": "dequant_gemm_pair_kernel",
            "dtype": "fp16 operands (weights dequantized to fp16, bf16 tokens converted), f32 accumulate",
            "clocks": merge_clocks(clocks)}


def run_gemv(args):
    """--workload gemv: config 2 alone (one GPU, or independent replicas on N)."""
    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback for the GPU arm)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    stream = torch.cuda.Stream(device=dev)
    peaks = measured_peaks()
    ps = ProjectionSet(dev, args.bits, args.groupsize, args.layers, args.seed + 1000 * rank, max_m=args.batch)
    top = ps.measure(args.batch, args.group, args.steps, args.warmup, stream, e2e=True)
    t = torch.tensor([top["ms_per_step"], ps.total_bytes / top["e2e"]["value"] / 1e6], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    sec, sec_e2e = float(t[0]) / 1e3, float(t[1]) / 1e3
    per_gpu = ps.total_bytes / sec / 1e9
    traffic = None
    if args.bits == 2 and args.groupsize == 128 and args.batch == 1:
        traffic = NCU_TRAFFIC_RATIO * ps.total_bytes / max(1, top["launches_per_step"])
    line = {
        "metric": "hlq_gemv_gbs", "value": world * per_gpu, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "repeats": REPEATS, "ms_per_step": sec * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32 accumulate over fp16 activations, 1-bit planes",
        "data": "synthetic",
        "config": {"workload": f"llama3-8b projection set w{args.bits}g{args.groupsize}, batch {args.batch}, "
                               f"{args.layers} layers", "grouping": args.group,
                   "l2": "weights per step larger than L2; no flush needed"},
        "pct_of_8tbs_per_gpu": 100.0 * per_gpu / HBM_NOMINAL_GBS,
        "algorithmic_bytes_per_step": ps.total_bytes, "clocks": top["clocks"],
        "e2e": {"value": world * ps.total_bytes / sec_e2e / 1e9, "unit": "GB/s",
                "h2d_bytes_per_step": top["e2e"]["h2d_bytes_per_step"],
                "d2h_bytes_per_step": top["e2e"]["d2h_bytes_per_step"]},
        "gpu_launches": int(top["launches_per_step"] * args.steps * REPEATS),
        "roofline": {"bound": "hbm", "achieved": per_gpu, "peak": peaks["hbm"], "unit": "GB/s",
                     "frac": per_gpu / peaks["hbm"], "traffic": traffic,
                     "traffic_source": "ncu capture of a 2-layer launch, scaled by algorithmic bytes",
                     "peak_source": f"of {peaks['kind']}",
                     "kernel": "batch_mma_kernel" if (args.batch >= 3 and args.bits in (2, 3)) else "lut8_gemv_kernel",
                     "launches_per_step": int(top["launches_per_step"]),
                     "avg_launch_us": sec * 1e6 / max(1, top["launches_per_step"])},
        "error_measure": NORMWISE,
    }
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


# ------------------------------------------------------------------------------------------
# GPU arm: whole-token decode, tensor-parallel over the ranks (config 5; the default)
# ------------------------------------------------------------------------------------------
def tp_parity(dec, dev, world):
    """One row-parallel projection through the GEMV with the fused all-reduce and through
    GEMV + NCCL all-reduce, fp32 outputs: the in-run evidence that the sharded path is right."""
    import torch
    import torch.distributed as dist
    from elutq_b200.linear import linear_forward
    L0 = dec.layers[0]
    w = L0["o"]
    i = w.info
    gen = torch.Generator(device=dev)
    gen.manual_seed(1234 + dec.rank)
    x = torch.randn((1, i.in_channel), device=dev, generator=gen).half()
    ref = linear_forward(x, w, dec.ws, out_dtype=torch.float32).clone()
    dist.all_reduce(ref)
    errs = []
    for _ in range(4):                                  # both slot parities, several launch numbers
        y = torch.full((1, i.out_channel), float("nan"), dtype=torch.float32, device=dev)
        dec.comm.forward(x, w, dec.ws, y)
        torch.cuda.synchronize()
        errs.append(float((y - ref).abs().max() / ref.abs().max()))
    t = torch.tensor([max(errs)], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    assert dec.ws.kernel_status() == 0
    return {"max_normwise_err": float(t[0]), "gate": 1e-5, "projection": f"o {i.out_channel}x{i.in_channel * world} "
            f"split over {world} ranks, fp32 outputs", "against": "LUT GEMV + NCCL all-reduce"}


def run_decode(args):
    import torch
    import torch.distributed as dist
    from elutq_b200.decoder import PRESETS, TPDecoder

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback for the GPU arm)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    cfg = PRESETS[args.model]
    if args.decode_layers:
        cfg = dataclasses.replace(cfg, layers=args.decode_layers)
    cfg = dataclasses.replace(cfg, bits=args.bits, groupsize=args.groupsize)
    fused = world > 1 and not args.nccl_allreduce
    dec = TPDecoder(cfg, dev, rank, world, seed=args.seed, grouped=not args.ungrouped,
                    fused_allreduce=fused, fused_glue=not args.torch_glue,
                    chain=not (args.launch_per_op or args.nccl_allreduce or args.torch_glue or args.ungrouped))
    parity = None
    if world > 1 and fused:
        parity = tp_parity(dec, dev, world)
        if parity["max_normwise_err"] > parity["gate"]:
            raise SystemExit(f"tensor-parallel parity failed: {parity}")
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
    stream = torch.cuda.current_stream(dev)
    ms, clocks = timed_blocks(graph.replay, args.steps, barrier, stream, local)
    # end to end: the token id comes from pinned host memory and the next token goes back to it
    tok_in = torch.ones(1, dtype=torch.int64).pin_memory()
    tok_out = torch.zeros(1, dtype=torch.int64).pin_memory()

    def e2e_step():
        dec.token.copy_(tok_in, non_blocking=True)
        graph.replay()
        tok_out.copy_(dec.next_token, non_blocking=True)
        stream.synchronize()
    ms2, _ = timed_blocks(e2e_step, args.steps, barrier, stream, local, 3)
    t = torch.tensor(ms + ms2, dtype=torch.float64, device=dev)
    lb = torch.tensor([float(dec.linear_bytes)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)         # every block: the slowest rank's time
        dist.all_reduce(lb, op=dist.ReduceOp.SUM)
    blocks = [float(v) for v in t[:len(ms)]]
    sec = statistics.median(blocks) / 1e3 / args.steps
    sec_e2e = statistics.median([float(v) for v in t[len(ms):]]) / 1e3 / args.steps
    assert dec.ws.kernel_status() == 0 and (not dec.fused_glue or dec.attn.status() == 0)
    assert dec.chain is None or dec.chain.status() == 0
    peaks = measured_peaks()
    my_bytes = float(dec.linear_bytes)
    launches = dec.launches_per_step()
    gemv_launches = 2 if dec.use_chain else len(dec.layers) * (4 if dec.grouped else 7) + 1
    line = {
        "metric": "decode_tokens_per_s", "value": 1.0 / sec, "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "repeats": REPEATS, "ms_per_step": sec * 1e3,
        "ms_per_step_min": min(blocks) / args.steps, "ms_per_step_max": max(blocks) / args.steps,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32 accumulate over fp16 activations, 1-bit planes; fp16 between the ops",
        "data": "synthetic",
        "config": decode_config(args.model, cfg, world,
                                "PyTorch glue ops (parity reference)" if args.torch_glue else
                                (DECODE_PATH if dec.use_chain else PER_OP_PATH)),
        "e2e": {"value": 1.0 / sec_e2e, "unit": "tokens/s", "h2d_bytes_per_step": 8, "d2h_bytes_per_step": 8},
        "gpu_launches": int(launches * args.steps * REPEATS),
        "launches_per_step": int(launches),
        "linear_algorithmic_bytes_per_token": float(lb[0]),
        "linear_gbs_over_step_time": float(lb[0]) / sec / 1e9,
        "pct_of_8tbs_per_gpu": 100.0 * my_bytes / sec / 1e9 / HBM_NOMINAL_GBS,
        "roofline": {"bound": "hbm", "achieved": my_bytes / sec / 1e9, "peak": peaks["hbm"], "unit": "GB/s",
                     "frac": my_bytes / sec / 1e9 / peaks["hbm"],
                     "traffic": (NCU_TRAFFIC_RATIO_CHAIN if dec.use_chain else NCU_TRAFFIC_RATIO) * my_bytes / gemv_launches,
                     "traffic_source": "ncu capture of a 4-layer launch of the kernel (profiles/), scaled by algorithmic bytes",
                     "peak_source": f"of {peaks['kind']}",
                     "kernel": "decode_chain_kernel" if dec.use_chain else "lut8_gemv_kernel",
                     "launches_per_step": gemv_launches,
                     "note": "achieved = this rank's linear bytes per token over the WHOLE step time (norms, "
                             "attention, collectives and launch gaps included), a lower bound of the kernel's own "
                             "rate; the kernel alone on the 8B set is under `gemv`"},
        "error_measure": NORMWISE,
        "clocks": merge_clocks(clocks),
    }
    if parity is not None:
        line["tp_parity"] = parity
    if world > 1:
        dist.barrier()
    if rank == 0:
        if world == 1 and not args.no_extras:
            dec.graph = None
            del graph
            side = torch.cuda.Stream(device=dev)
            line["gemv"], _ = gemv_object(dev, args, side, max(args.steps, 20), max(args.warmup, 5))
            line["batches"] = batches_object(dev, args, side, max(args.steps, 20), 3)
            line["prefill"] = prefill_object(dev, args, 2, 5, 3)
        if world == 1 and not args.skip_cpu:
            from oracle import build as obuild
            obuild.build()
            cores = host_cores()
            sample = CpuDecodeSample(cfg, min(args.cpu_layers, cfg.layers), cores, seed=args.seed)
            r = sample.run(args.cpu_steps, 2)
            line["cpu_baseline"] = {"value": r["tokens_per_s"], "unit": "tokens/s", "cores": max(sample.threads_used),
                                    "kind": "port", "sample": sample.describe() + f"; {args.cpu_steps} passes",
                                    "host_cores": cores, "cpu_model": cpu_model(), "linear_gbs": r["gbs"],
                                    "config1_single_gemv": cpu_config1(cores)}
        print(json.dumps(line), flush=True)
    if world > 1:
        # a communicator cannot be torn down while a captured graph still holds its kernels
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        os._exit(0)


def run_prefill(args):
    import torch
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    p = prefill_object(dev, args, args.prefill_layers, args.steps, args.warmup)
    peaks = measured_peaks()
    print(json.dumps({
        "metric": "hlq_prefill_tflops", "value": p["value"], "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": p["ms_per_step"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": p["dtype"], "data": "synthetic", "config": {"workload": p["workload"]},
        "gpu_launches": int(p["launches_per_step"] * args.steps * 3), "clocks": p["clocks"],
        "roofline": {"bound": "tensor", "achieved": p["value"], "peak": peaks["tf_sustained"], "unit": "TFLOP/s",
                     "frac": p["frac_of_sustained_bf16"], "frac_of_burst": p["frac_of_burst_bf16"], "traffic": None,
                     "peak_source": f"of {peaks['kind']}, sustained", "kernel": "dequant_gemm_pair_kernel"}}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="decode", choices=["decode", "gemv", "prefill"])
    ap.add_argument("--bits", type=int, default=2)
    ap.add_argument("--groupsize", type=int, default=128)
    ap.add_argument("--seed", type=int, default=0)
    # decode
    ap.add_argument("--model", default="llama3-70b", help="decoder preset")
    ap.add_argument("--decode-layers", type=int, default=0, help="override the preset's layer count")
    ap.add_argument("--ungrouped", action="store_true", help="one launch per projection")
    ap.add_argument("--torch-glue", action="store_true", help="PyTorch ops between the linears")
    ap.add_argument("--nccl-allreduce", action="store_true",
                    help="NCCL all-reduce after o and down instead of the one fused into the GEMV kernel")
    ap.add_argument("--launch-per-op", action="store_true",
                    help="one launch per op (8 per layer) instead of the decode chain (one persistent kernel)")
    ap.add_argument("--no-graph", action="store_true", help="launch from the host every step")
    ap.add_argument("--no-extras", action="store_true", help="N = 1: skip the gemv / batches / prefill objects")
    # projection set (gemv object and --workload gemv)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--layers", type=int, default=32, help="layers of the 8B projection set")
    ap.add_argument("--group", default="model", choices=["none", "layer4", "model"])
    # prefill
    ap.add_argument("--tokens", type=int, default=2048, help="prefill: rows of activations")
    ap.add_argument("--prefill-layers", type=int, default=2)
    # CPU legs
    ap.add_argument("--cpu-layers", type=int, default=1, help="decoder layers in the CPU sample")
    ap.add_argument("--cpu-steps", type=int, default=5)
    ap.add_argument("--skip-cpu", action="store_true")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "gemv":
        run_gemv(args)
    elif args.workload == "prefill":
        run_prefill(args)
    else:
        run_decode(args)


if __name__ == "__main__":
    main()
