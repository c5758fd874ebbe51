#!/usr/bin/env python
"""Benchmark of the quantized-contraction hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload decode_gemv] [--impl ours|reference]

One JSON line on stdout (rank 0).  Workloads (synthetic, seeded; shapes from the decode /
prefill configurations of the Gemma-4 12B-like model):

  decode_gemv   48 "layers" x {gate/up 3840->30720, down 15360->3840, QKV 3840->8192,
                O 4096->3840}: FP8 E4M3 weights with bf16 per-row scales, bf16 activations
                quantised per token to E4M3 inside each GEMV launch; 48 distinct weight sets
                (10.76 GB, far larger than L2).  Metric: GB/s of algorithmic bytes.

  nvfp4_linear  (reported under "other_workloads") X bf16 [512, 3840] -> NVFP4 quantiser -> tcgen05 GEMM
                against W NVFP4 [15360, 3840]; eight distinct weight sets (266 MB > L2) in rotation.
                Metric: TFLOP/s counting the GEMM's 2*M*N*K flops, for the GEMM alone and with the
                activation quantiser in the timed region.
  moe_layer     (reported under "other_workloads") one 26B-A4B-like MoE layer on 4096 tokens: router,
                top-8, stable permutation, dispatch, grouped NVFP4 expert GEMMs, GELU requantisation,
                shared FFN, slot-ordered combine.  Metric: tokens/s.

A step is one pass over all 48 layers, replayed as one CUDA graph.  `value` is measured with
inputs resident in HBM; `e2e` copies the step's activations from pinned host memory and the
results back inside the timed region.  With N > 1 every rank runs an independent replica
(the path does not shard at batch 1) and `value` is the sum over ranks.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

DECODE_SHAPES = [("gate_up", 30720, 3840), ("down", 3840, 15360), ("qkv", 8192, 3840), ("o", 3840, 4096)]
LAYERS = 48
SEED = 20261125


# dram__bytes_read.sum + dram__bytes_write.sum of the captured fp8_gemv_kernel launches divided by
# their algorithmic bytes (profiles/fp8_gemv_kernel_decode.md).
NCU_TRAFFIC_OVER_ALGORITHMIC = 1.00


def decode_bytes_per_layer() -> int:
    """Algorithmic bytes of one layer: weights + fp32-equivalent scales + bf16 x + bf16 y."""
    total = 0
    for _, rows, k in DECODE_SHAPES:
        total += rows * k + rows * 4 + k * 2 + rows * 2
    return total


def measured_peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.samples: list[list[str]] = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) == 6:
                self.samples.append(parts)

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        mhz = sorted(int(s[0]) for s in self.samples if s[0].isdigit())
        reasons = set()
        for s in self.samples:
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), s[2:]):
                if v == "Active":
                    reasons.add(name)
        mx = [int(s[1]) for s in self.samples if s[1].isdigit()]
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(self.samples)}


# --------------------------------------------------------------------------------------------
# reference arm / CPU baseline: the reference's own CPU numeric path on a bounded sample
# --------------------------------------------------------------------------------------------
def cpu_decode_sample(steps: int, warmup: int, use_ref: bool):
    """Times one decode layer (all four GEMVs incl. the per-token FP8 quantisation) on the host
    cores with the reference's src/numeric/fp8.cpp functions (or the oracle port when the
    compiled reference is absent).  Returns (GB/s, seconds per sample, cores, kind)."""
    import numpy as np
    from oracle import Oracle, default_threads, ref_available
    kind = "reference" if use_ref and ref_available() else "port"
    o = Oracle(ref=(kind == "reference"))
    port = Oracle()
    threads = default_threads()
    rng = np.random.default_rng(SEED)
    layer = []
    for _, rows, k in DECODE_SHAPES:
        w = rng.integers(0, 256, size=(rows, k), dtype=np.uint8)
        w[(w & 0x7F) == 0x7F] = 0x38
        ws = port.to_bf16(rng.uniform(1e-4, 2e-4, size=rows).astype(np.float32))
        x = port.from_bf16(port.to_bf16(rng.standard_normal((1, k)).astype(np.float32)))
        layer.append((x, w, ws))

    def one_pass():
        for x, w, ws in layer:
            q, s = o.fp8_quantize(x, threads=threads)
            o.fp8_matmul(q, s, w, ws, threads=threads)

    for _ in range(warmup):
        one_pass()
    t0 = time.perf_counter()
    for _ in range(steps):
        one_pass()
    dt = (time.perf_counter() - t0) / steps
    return decode_bytes_per_layer() / dt / 1e9, dt, threads, kind


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    gbs, dt, cores, kind = cpu_decode_sample(args.steps, min(args.warmup, 1), use_ref=True)
    sample = "one decode layer (4 FP8 GEMVs + per-token quantisation, 224 MB) per step, all host cores"
    line = {
        "impl": "reference", "metric": "decode GEMV GB/s", "value": gbs, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "fp8_e4m3", "data": "synthetic",
        "config": {"workload": "decode_gemv", "layers": LAYERS, "shapes": DECODE_SHAPES},
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------------
# our arm
# --------------------------------------------------------------------------------------------
def run_decode_gemv(args):
    import torch
    import torch.distributed as dist
    from gem16_b200 import load

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    lib = load()
    lib.gemb_device_check()

    # ---- synthetic model state: 48 distinct FP8 weight sets quantised with our own quantizer --
    gen = torch.Generator(device=dev)
    gen.manual_seed(SEED + 1000 * 1 + rank)
    weights = []
    layers = args.layers
    for layer in range(layers):
        mats = []
        for _, rows, k in DECODE_SHAPES:
            w = torch.randn((rows, k), device=dev, dtype=torch.float32, generator=gen) * 0.02
            wq = torch.empty((rows, k), device=dev, dtype=torch.uint8)
            wsc = torch.empty((rows,), device=dev, dtype=torch.float32)
            lib.gemb_fp8_quantize(w, 0, wq, wsc, rows, k, None)
            mats.append((wq, wsc.to(torch.bfloat16).view(torch.int16)))
            del w
        weights.append(mats)
    # activations: one bf16 vector per op, in one contiguous buffer (device + pinned host copy)
    x_elems = sum(k for _, _, k in DECODE_SHAPES) * layers
    y_elems = sum(r for _, r, _ in DECODE_SHAPES) * layers
    x_host = torch.randn((x_elems,), dtype=torch.float32).to(torch.bfloat16).pin_memory()
    y_host = torch.empty((y_elems,), dtype=torch.bfloat16).pin_memory()
    x_dev = x_host.to(dev)
    y_dev = torch.zeros((y_elems,), device=dev, dtype=torch.bfloat16)

    # "fused": one launch per projection, the bf16 activation is quantised inside the GEMV.
    # "split": the decode-size token quantizer, then the GEMV on E4M3 bytes (fp32 out); with
    # programmatic dependent launch the GEMV prefetches weights while the quantizer runs.
    split = args.decode_path == "split"
    xq_dev = torch.empty((x_elems,), dtype=torch.uint8, device=dev)
    xs_dev = torch.empty((layers * len(DECODE_SHAPES),), device=dev)
    y32_dev = torch.zeros((y_elems,), device=dev) if split else None
    y_host32 = torch.empty((y_elems,), dtype=torch.float32).pin_memory() if split else None

    def enqueue_pass():
        xo = yo = 0
        n = 0
        st = torch.cuda.current_stream()
        for mats in weights:
            for (wq, ws), (_, rows, k) in zip(mats, DECODE_SHAPES):
                if split:
                    lib.gemb_fp8_quantize(x_dev[xo:xo + k], 1, xq_dev[xo:xo + k], xs_dev[n:n + 1], 1, k, st)
                    lib.gemb_fp8_gemv(xq_dev[xo:xo + k], xs_dev[n:n + 1], wq, ws, y32_dev[yo:yo + rows], rows, k, st)
                else:
                    lib.gemb_fp8_gemv_bf16in(x_dev[xo:xo + k], wq, ws, y_dev[yo:yo + rows], 1, rows, k, st)
                xo += k
                yo += rows
                n += 1
        return n * (2 if split else 1)

    def enqueue_gemvs_only():
        # The same projections on the already quantised activations: the dominant kernel alone,
        # for the roofline object (its launches are 99.9 % of the bytes of a pass).
        xo = yo = n = 0
        st = torch.cuda.current_stream()
        for mats in weights:
            for (wq, ws), (_, rows, k) in zip(mats, DECODE_SHAPES):
                lib.gemb_fp8_gemv(xq_dev[xo:xo + k], xs_dev[n:n + 1], wq, ws, y32_dev[yo:yo + rows], rows, k, st)
                xo += k
                yo += rows
                n += 1
        return n

    stream = torch.cuda.Stream(device=dev)
    with torch.cuda.stream(stream):
        launches_per_step = enqueue_pass()  # also warms lazily initialised state before capture
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            enqueue_pass()
        gemv_graph = None
        gemv_launches = 0
        if split:
            gemv_launches = enqueue_gemvs_only()
            stream.synchronize()
            gemv_graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gemv_graph, stream=stream):
                enqueue_gemvs_only()

        def barrier():
            torch.cuda.synchronize(dev)
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize(dev)

        def timed(fn, steps):
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            barrier()
            start.record(stream)
            for _ in range(steps):
                fn()
            end.record(stream)
            barrier()
            ms = start.elapsed_time(end)
            if world > 1:
                t = torch.tensor([ms], device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms = float(t.item())
            return ms / 1e3

        def step_resident():
            graph.replay()

        def step_e2e():
            x_dev.copy_(x_host, non_blocking=True)
            graph.replay()
            (y_host32 if split else y_host).copy_(y32_dev if split else y_dev, non_blocking=True)
            stream.synchronize()

        for _ in range(max(args.warmup, 3)):
            step_resident()
        sampler = ClockSampler(local)
        if rank == 0:
            sampler.start()
        secs = timed(step_resident, args.steps)
        clocks = sampler.stop() if rank == 0 else None
        for _ in range(2):
            step_e2e()
        secs_e2e = timed(step_e2e, args.steps)
        secs_gemv = None
        if gemv_graph is not None:
            for _ in range(3):
                gemv_graph.replay()
            secs_gemv = timed(gemv_graph.replay, args.steps)

    bytes_step = decode_bytes_per_layer() * layers
    value = world * bytes_step * args.steps / secs / 1e9
    e2e = world * bytes_step * args.steps / secs_e2e / 1e9
    moe_ep = tp_mlp = None
    if not args.no_other_workloads:
        del weights, graph, gemv_graph
        torch.cuda.empty_cache()
        try:   # collective: every rank takes part
            moe_ep = bench_moe_ep(lib, dev, world, rank)
        except Exception as exc:
            moe_ep = {"error": f"{type(exc).__name__}: {exc}"}
        if world > 1:
            try:
                tp_mlp = bench_tp_mlp(lib, dev, world, rank)
            except Exception as exc:
                tp_mlp = {"error": f"{type(exc).__name__}: {exc}"}
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    peaks = measured_peaks()
    # Roofline of the dominant kernel: algorithmic bytes of one GEMV launch (its weight matrix, the
    # bf16 row scales, the activation and the output; the pass total / launches) over that kernel's
    # average launch duration, timed with CUDA events over a region that launches only it.
    if secs_gemv is not None:
        launch_s = secs_gemv / (args.steps * gemv_launches)
        achieved = bytes_step / gemv_launches / launch_s / 1e9
    else:
        launch_s = secs / (args.steps * launches_per_step)
        achieved = bytes_step / launches_per_step / launch_s / 1e9
    whole_pass = bytes_step * args.steps / secs / 1e9 if world == 1 else value / world
    line = {
        "metric": "decode GEMV GB/s", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": secs / args.steps * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "fp8_e4m3 (fp32 accumulate)", "data": "synthetic",
        "config": {"workload": "decode_gemv", "layers": layers, "shapes": DECODE_SHAPES,
                   "l2": f"{layers} distinct weight sets, {bytes_step / 1e9:.2f} GB per pass >> 126 MB L2",
                   "multi_gpu": "replicas only", "decode_path": args.decode_path},
        "e2e": {"value": e2e, "unit": "GB/s", "h2d_bytes_per_step": x_elems * 2, "d2h_bytes_per_step": y_elems * (4 if split else 2)},
        "gpu_launches": launches_per_step * args.steps,
        "clocks": clocks,
        "roofline": {"bound": "hbm", "kernel": "fp8_gemv_kernel" + ("" if split else " (bf16-in fused quantisation)"),
                     "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / peaks["hbm_gbs"], "peak_source": peaks["source"],
                     "frac_of_nominal_8TBs": achieved / 8000.0,
                     # dram read + write bytes per launch from the committed ncu capture of this kernel
                     # (profiles/fp8_gemv_kernel_decode.md), as a ratio to the algorithmic bytes
                     "traffic": NCU_TRAFFIC_OVER_ALGORITHMIC * bytes_step / (gemv_launches if secs_gemv is not None else launches_per_step),
                     "traffic_unit": "bytes per launch (average)",
                     "algorithmic_bytes_per_launch": bytes_step / (gemv_launches if secs_gemv is not None else launches_per_step),
                     "avg_launch_us": launch_s * 1e6,
                     "whole_pass": {"kernels": "fp8_quantize_decode_kernel + fp8_gemv_kernel" if split else "fp8_gemv_kernel",
                                    "achieved": whole_pass, "frac": whole_pass / peaks["hbm_gbs"],
                                    "launches_per_pass": launches_per_step}},
    }
    if moe_ep is not None:
        line["other_workloads"] = {"moe_ep_stack": moe_ep}
        if tp_mlp is not None:
            line["other_workloads"]["tp_mlp"] = tp_mlp
    if world == 1 and not args.no_other_workloads:
        other = line["other_workloads"]
        for name, fn in (("nvfp4_linear", bench_nvfp4_linear), ("prefill_gemm", bench_prefill_gemm),
                         ("prefill_stack", bench_prefill_stack), ("moe_layer", bench_moe_layer),
                         ("output_head", bench_output_head), ("verifier_gemv", bench_verifier_gemv)):
            try:
                other[name] = fn(lib, dev)
            except Exception as exc:  # a secondary workload must not take the headline line down
                other[name] = {"error": f"{type(exc).__name__}: {exc}"}
    if world == 1 and not args.no_cpu_baseline:
        gbs, dt, cores, kind = cpu_decode_sample(1, 0, use_ref=True)
        line["cpu_baseline"] = {"value": gbs, "unit": "GB/s", "cores": cores, "kind": kind,
                                "sample": f"one decode layer of 48 (224 MB), {dt:.2f} s on {cores} host threads"}
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# --------------------------------------------------------------------------------------------
# secondary workloads (rank 0 only, N = 1 semantics; reported under "other_workloads")
# --------------------------------------------------------------------------------------------
def graph_time(enqueue, launches_per_graph, reps=20):
    """Seconds per enqueue() pass, replayed as one CUDA graph, timed with CUDA events."""
    import torch
    st = torch.cuda.Stream()
    with torch.cuda.stream(st):
        enqueue(st)
        st.synchronize()
        # Captured twice: a graph with a forked side stream instantiated right after the eager pass
        # has replayed measurably slower here than the same capture taken once more.
        for _ in range(2):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=st):
                enqueue(st)
            for _ in range(5):
                g.replay()
            st.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        st.synchronize()
        s.record(st)
        for _ in range(reps):
            g.replay()
        e.record(st)
        st.synchronize()
    return s.elapsed_time(e) / reps / 1e3


def bench_nvfp4_linear(lib, dev):
    import torch
    m, n, k, copies = 512, 15360, 3840, 8
    gen = torch.Generator(device=dev)
    gen.manual_seed(SEED)
    x = torch.randn((m, k), device=dev, generator=gen).to(torch.bfloat16)
    ga = float(2688.0 / x.float().abs().max().item())
    xq = torch.empty((m, k // 2), dtype=torch.uint8, device=dev)
    xs = torch.zeros((lib.cdll.gemb_interleaved_scale_bytes(m, k),), dtype=torch.uint8, device=dev)
    ws = []
    for _ in range(copies):
        w = torch.randn((n, k), device=dev, generator=gen) * 0.02
        gw = float(2688.0 / w.abs().max().item())
        wq = torch.empty((n, k // 2), dtype=torch.uint8, device=dev)
        wsc = torch.zeros((lib.cdll.gemb_interleaved_scale_bytes(n, k),), dtype=torch.uint8, device=dev)
        lib.gemb_nvfp4_quantize(w, 0, wq, wsc, n, k, gw, 1, 0, None)
        ws.append((wq, wsc, gw))
        del w
    out = torch.empty((m, n), dtype=torch.int16, device=dev)
    lib.gemb_nvfp4_quantize(x.view(torch.int16), 1, xq, xs, m, k, ga, 1, 0, None)

    def gemm_only(st):
        for wq, wsc, gw in ws:
            lib.gemb_nvfp4_gemm_bf16(xq, xs, wq, wsc, out, m, n, k, ga, gw, st)

    def quant_and_gemm(st):
        for wq, wsc, gw in ws:
            lib.gemb_nvfp4_quantize(x.view(torch.int16), 1, xq, xs, m, k, ga, 1, 0, st)
            lib.gemb_nvfp4_gemm_bf16(xq, xs, wq, wsc, out, m, n, k, ga, gw, st)

    t_gemm = graph_time(gemm_only, copies) / copies
    t_both = graph_time(quant_and_gemm, 2 * copies) / copies
    lib.gemb_check_device_status()
    flops = 2.0 * m * n * k
    nominal = 9000.0
    return {"metric": "NVFP4 GEMM TFLOP/s", "workload": "nvfp4_linear 512x15360x3840 (W4A4)",
            "value": flops / t_gemm / 1e12, "unit": "TFLOP/s", "us_per_linear": t_gemm * 1e6,
            "with_activation_quantizer": {"value": flops / t_both / 1e12, "us_per_linear": t_both * 1e6},
            "roofline": {"bound": "tensor", "kernel": "gemm_kernel<nvfp4, 256x256 on CTA pairs>", "achieved": flops / t_gemm / 1e12,
                         "peak": nominal, "unit": "TFLOP/s", "frac": flops / t_gemm / 1e12 / nominal,
                         "peak_source": "nominal dense FP4 (9 PFLOP/s); MEASURED_PEAKS.json has no FP4 figure",
                         "frac_of_4x_measured_bf16_sustained": flops / t_gemm / 1e12 / (4 * 1391.3)},
            "l2": f"{copies} distinct weight sets in rotation, {copies * (n * k // 2 + n * k // 16) / 1e6:.0f} MB > 126 MB L2"}


def bench_prefill_gemm(lib, dev):
    """The 16,384-token prefill projections of one 12B-like layer (shapes of the prefill stack):
    NVFP4 gate/up/down and FP8 QKV/O GEMMs on pre-quantised operands, each timed alone."""
    import torch
    m = 16384
    out = {"metric": "prefill GEMM TFLOP/s", "tokens": m, "gemms": {}}
    gen = torch.Generator(device=dev)
    gen.manual_seed(SEED + 2000)
    for name, n, k, fp4 in (("gate_or_up", 15360, 3840, True), ("down", 3840, 15360, True),
                            ("qkv", 8192, 3840, False), ("o", 3840, 4096, False)):
        x = torch.randn((m, k), device=dev, generator=gen).to(torch.bfloat16)
        w = (torch.randn((n, k), device=dev, generator=gen) * 0.02)
        y = torch.empty((m, n), dtype=torch.int16, device=dev)
        if fp4:
            ga, gw = float(2688.0 / x.float().abs().max().item()), float(2688.0 / w.abs().max().item())
            xq = torch.empty((m, k // 2), dtype=torch.uint8, device=dev)
            xs = torch.zeros((lib.cdll.gemb_interleaved_scale_bytes(m, k),), dtype=torch.uint8, device=dev)
            wq = torch.empty((n, k // 2), dtype=torch.uint8, device=dev)
            ws = torch.zeros((lib.cdll.gemb_interleaved_scale_bytes(n, k),), dtype=torch.uint8, device=dev)
            lib.gemb_nvfp4_quantize(x.view(torch.int16), 1, xq, xs, m, k, ga, 1, 0, None)
            lib.gemb_nvfp4_quantize(w, 0, wq, ws, n, k, gw, 1, 0, None)
            fn = lambda st: lib.gemb_nvfp4_gemm_bf16(xq, xs, wq, ws, y, m, n, k, ga, gw, st)
            peak = 9000.0
        else:
            xq = torch.empty((m, k), dtype=torch.uint8, device=dev)
            xs = torch.empty((m,), device=dev)
            wq = torch.empty((n, k), dtype=torch.uint8, device=dev)
            ws = torch.empty((n,), device=dev)
            lib.gemb_fp8_quantize(x.view(torch.int16), 1, xq, xs, m, k, None)
            lib.gemb_fp8_quantize(w, 0, wq, ws, n, k, None)
            wsb = ws.to(torch.bfloat16).view(torch.int16)
            fn = lambda st: lib.gemb_fp8_gemm_bf16(xq, xs, wq, wsb, y, m, n, k, st)
            peak = 4500.0
        del x, w
        secs = graph_time(fn, 1, reps=10)
        tf = 2.0 * m * n * k / secs / 1e12
        out["gemms"][name] = {"rows": n, "k": k, "format": "nvfp4" if fp4 else "fp8", "us": secs * 1e6, "tflops": tf,
                              "frac_of_nominal_dense_peak": tf / peak}
    lib.gemb_check_device_status()
    return out


def bench_prefill_stack(lib, dev, layers=48, tokens=16384):
    """Dense 12B-like prefill linear stack: per layer FP8 QKV and O projections and the NVFP4 gated
    MLP, every activation quantiser inside the timed region (attention itself is replaced by a
    seeded bf16 tensor: it is not part of this path)."""
    import torch
    h, qkv, ao, inter = 3840, 8192, 4096, 15360
    gen = torch.Generator(device=dev)
    gen.manual_seed(SEED + 2500)
    c = lib.cdll

    def fp8_w(n, k):
        w = torch.randn((n, k), device=dev, generator=gen) * 0.02
        q = torch.empty((n, k), dtype=torch.uint8, device=dev)
        s = torch.empty((n,), device=dev)
        lib.gemb_fp8_quantize(w, 0, q, s, n, k, None)
        return q, s.to(torch.bfloat16).view(torch.int16)

    def fp4_w(n, k):
        w = torch.randn((n, k), device=dev, generator=gen) * 0.02
        g = float(2688.0 / w.abs().max().item())
        q = torch.empty((n, k // 2), dtype=torch.uint8, device=dev)
        s = torch.zeros((c.gemb_interleaved_scale_bytes(n, k),), dtype=torch.uint8, device=dev)
        lib.gemb_nvfp4_quantize(w, 0, q, s, n, k, g, 1, 0, None)
        return q, s, g

    weights = [(fp8_w(qkv, h), fp8_w(h, ao), fp4_w(inter, h), fp4_w(inter, h), fp4_w(h, inter)) for _ in range(layers)]
    x = torch.randn((tokens, h), device=dev, generator=gen).to(torch.bfloat16).view(torch.int16)
    attn = torch.randn((tokens, ao), device=dev, generator=gen).to(torch.bfloat16).view(torch.int16)
    u8 = dict(dtype=torch.uint8, device=dev)
    xq, xs = torch.empty((tokens, h), **u8), torch.empty((tokens,), device=dev)
    aq, as_ = torch.empty((tokens, ao), **u8), torch.empty((tokens,), device=dev)
    y_qkv = torch.empty((tokens, qkv), dtype=torch.int16, device=dev)
    y_o = torch.empty((tokens, h), dtype=torch.int16, device=dev)
    oq = torch.empty((tokens, h // 2), **u8)
    os_ = torch.zeros((c.gemb_interleaved_scale_bytes(tokens, h),), **u8)
    gate = torch.empty((tokens, inter), dtype=torch.int16, device=dev)
    up = torch.empty((tokens, inter), dtype=torch.int16, device=dev)
    pq = torch.empty((tokens, inter // 2), **u8)
    ps = torch.zeros((c.gemb_interleaved_scale_bytes(tokens, inter),), **u8)
    out = torch.empty((tokens, h), dtype=torch.int16, device=dev)
    ga_mlp, ga_dn = 2688.0 / 0.6, 2688.0 / 0.05   # static input divisors (checkpoint-style constants)

    def run(st):
        for (wq, wqs), (wo, wos), (wg, wgs, gg), (wu, wus, gu), (wd, wds, gd) in weights:
            lib.gemb_fp8_quantize(x, 1, xq, xs, tokens, h, st)
            lib.gemb_fp8_gemm_bf16(xq, xs, wq, wqs, y_qkv, tokens, qkv, h, st)
            lib.gemb_fp8_quantize(attn, 1, aq, as_, tokens, ao, st)
            lib.gemb_fp8_gemm_bf16(aq, as_, wo, wos, y_o, tokens, h, ao, st)
            lib.gemb_nvfp4_quantize(y_o, 1, oq, os_, tokens, h, ga_mlp, 1, 0, st)
            lib.gemb_nvfp4_gemm_bf16(oq, os_, wg, wgs, gate, tokens, inter, h, ga_mlp, gg, st)
            lib.gemb_nvfp4_gemm_bf16(oq, os_, wu, wus, up, tokens, inter, h, ga_mlp, gu, st)
            lib.gemb_nvfp4_gated_gelu_quantize(gate, up, 1, pq, ps, tokens, inter, ga_dn, 1, 0, st)
            lib.gemb_nvfp4_gemm_bf16(pq, ps, wd, wds, out, tokens, h, inter, ga_dn, gd, st)

    secs = graph_time(run, 9 * layers, reps=3)
    lib.gemb_check_device_status()
    fp8_flops = 2.0 * tokens * (qkv * h + h * ao)
    fp4_flops = 2.0 * tokens * 3 * inter * h
    return {"metric": "prefill linear stack TFLOP/s", "workload": f"{layers} layers x 16,384 tokens: FP8 QKV+O, NVFP4 gate/up/down, quantisers timed",
            "ms_per_stack": secs * 1e3, "ms_per_layer": secs * 1e3 / layers, "tokens_per_s": tokens / secs,
            "tflops_total": (fp8_flops + fp4_flops) * layers / secs / 1e12,
            "flops_per_layer": {"fp8": fp8_flops, "nvfp4": fp4_flops},
            "ideal_ms_per_layer_at_nominal_peaks": (fp8_flops / 4.5e15 + fp4_flops / 9e15) * 1e3}


def bench_moe_layer(lib, dev, tokens=4096):
    import torch
    from gem16_b200.moe import MoeLayer, synthetic_weights
    w = synthetic_weights(dev, SEED + 3000)
    gen = torch.Generator(device=dev)
    gen.manual_seed(SEED + 3001)
    x = torch.randn((tokens, 2816), device=dev, generator=gen).to(torch.bfloat16)
    ga = float(2688.0 / x.float().abs().max().item())
    layer = MoeLayer(w, tokens, 8, ga, 2688.0 / 8.0, 2688.0 / 8.0)
    xi = x.view(torch.int16)
    secs = graph_time(lambda st: layer.forward(xi, st), 14)
    lib.gemb_check_device_status()
    flops = 2.0 * tokens * 128 * 2816 + tokens * 8 * 2.0 * 3 * 704 * 2816 + tokens * 2.0 * 3 * 2112 * 2816
    weight_bytes = 128 * 3 * 704 * 2816 * 0.5625 + 3 * 2112 * 2816 * 0.5625 + 128 * 2816 * 4
    return {"metric": "MoE layer tokens/s", "workload": f"moe_layer {tokens} tokens, 128 experts top-8, hidden 2816, expert 704, shared 2112",
            "value": tokens / secs, "unit": "tokens/s", "us_per_layer": secs * 1e6,
            "flops": flops, "achieved_tflops": flops / secs / 1e12, "weight_bytes": weight_bytes,
            "bounds_us": {"tensor_at_9PF": flops / 9e15 * 1e6, "hbm_weights_at_measured_peak": weight_bytes / (measured_peaks()["hbm_gbs"] * 1e9) * 1e6},
            "padded_rows": int(layer.plan[1].item()), "tiles": int(layer.plan[0].item()),
            "expert_count_max": int(layer.counts.max().item()), "expert_count_min": int(layer.counts.min().item())}


def bench_output_head(lib, dev, vocab=262144, hidden=3840):
    """Tied bf16 output head of one decode step: 262,144 x 3,840 bf16 = 2.0 GB read per launch (far
    beyond L2), fused soft cap + suppression + arg-max; one hidden row (decode) and five (the
    reference's speculative-decoding verifier)."""
    import torch
    gen = torch.Generator(device=dev)
    gen.manual_seed(SEED + 7000)
    w = (torch.randn((vocab, hidden), device=dev, generator=gen) * 0.05).to(torch.bfloat16).view(torch.int16)
    blocks = lib.cdll.gemb_output_head_candidate_blocks()
    peaks = measured_peaks()
    out = {"metric": "output head GB/s", "workload": f"output_head {vocab}x{hidden} bf16, soft cap 30, arg-max", "rows": {}}
    for rows in (1, 5):
        h = torch.randn((rows, hidden), device=dev, generator=gen)
        cand = torch.zeros((rows, blocks, 2), dtype=torch.int32, device=dev)
        sel = torch.zeros((rows,), dtype=torch.int32, device=dev)
        sup = torch.tensor([0, 1, 2, 3], dtype=torch.int32, device=dev)

        def step(st):
            lib.gemb_output_head_candidates(w, h, rows, sup, 4, None, cand, None, vocab, hidden, st)
            lib.gemb_output_head_argmax(cand, rows, sel, st)

        t = graph_time(step, 2)
        nbytes = vocab * hidden * 2 + rows * hidden * 4 + rows * blocks * 8
        out["rows"][str(rows)] = {"us": t * 1e6, "gbs": nbytes / t / 1e9, "frac_of_measured_hbm_peak": nbytes / t / 1e9 / peaks["hbm_gbs"]}
    return out


def bench_verifier_gemv(lib, dev, sets=6):
    """The decode projection set at the speculative-decoding verifier's batch sizes (3 and 5 tokens):
    small-batch FP8 GEMV, fp32 out, weights streamed once per launch; `sets` distinct weight sets in
    rotation (1.35 GB, far beyond L2)."""
    import torch
    gen = torch.Generator(device=dev)
    gen.manual_seed(SEED + 8000)
    weights = []
    for _ in range(sets):
        mats = []
        for _, rows, k in DECODE_SHAPES:
            w = torch.randn((rows, k), device=dev, generator=gen) * 0.02
            wq = torch.empty((rows, k), device=dev, dtype=torch.uint8)
            wsc = torch.empty((rows,), device=dev)
            lib.gemb_fp8_quantize(w, 0, wq, wsc, rows, k, None)
            mats.append((wq, wsc.to(torch.bfloat16).view(torch.int16)))
            del w
        weights.append(mats)
    peaks = measured_peaks()
    out = {"metric": "verifier GEMV GB/s", "workload": "decode projection set at 3 and 5 tokens, FP8, fp32 out", "tokens": {}}
    for tokens in (3, 5):
        acts = []
        for _, rows, k in DECODE_SHAPES:
            x = torch.randn((tokens, k), device=dev, generator=gen)
            xq = torch.empty((tokens, k), device=dev, dtype=torch.uint8)
            xs = torch.empty((tokens,), device=dev)
            lib.gemb_fp8_quantize(x, 0, xq, xs, tokens, k, None)
            acts.append((xq, xs, torch.zeros((tokens, rows), device=dev)))

        def step(st):
            for mats in weights:
                for (wq, ws), (xq, xs, y), (_, rows, k) in zip(mats, acts, DECODE_SHAPES):
                    lib.gemb_fp8_gemv_batch(xq, xs, wq, ws, y, tokens, rows, k, st)

        t = graph_time(step, sets * len(DECODE_SHAPES))
        nbytes = sets * sum(r * k + 2 * r + tokens * (k + 4 * r) for _, r, k in DECODE_SHAPES)
        out["tokens"][str(tokens)] = {"us_per_layer": t / sets * 1e6, "gbs": nbytes / t / 1e9,
                                      "frac_of_measured_hbm_peak": nbytes / t / 1e9 / peaks["hbm_gbs"]}
    return out


def bench_tp_mlp(lib, dev, world, rank, tokens=16384):
    """Tensor-parallel 12B-like gated MLP (hidden 3840, intermediate 15360) on 16,384 tokens: gate/up
    column split, down row split with an fp32 all-reduce.  Collective; N = 1 runs it unsharded."""
    import torch
    import torch.distributed as dist
    from gem16_b200.tp import TpMlp
    hidden, inter = 3840, 15360
    gen = torch.Generator(device=dev)
    gen.manual_seed(SEED + 5000)

    def quant(rows, k):
        w = torch.randn((rows, k), device=dev, generator=gen) * 0.02
        div = float(2688.0 / w.abs().max().item())
        p = torch.empty((rows, k // 2), dtype=torch.uint8, device=dev)
        s = torch.empty((rows, k // 16), dtype=torch.uint8, device=dev)
        lib.gemb_nvfp4_quantize(w, 0, p, s, rows, k, div, 0, 0, None)
        return p, s, div

    gate, up, down = quant(inter, hidden), quant(inter, hidden), quant(hidden, inter)
    x = torch.randn((tokens, hidden), device=dev, generator=gen).to(torch.bfloat16).view(torch.int16)
    if world == 1 and not dist.is_initialized():
        dist.init_process_group("nccl", init_method="tcp://127.0.0.1:29577", rank=0, world_size=1, device_id=dev)
    mlp = TpMlp(dev, gate, up, down, tokens, 700.0, 2688.0 / 0.05)
    del gate, up, down
    for _ in range(3):
        mlp.forward(x)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = 10
    s.record()
    for _ in range(reps):
        mlp.forward(x)
    e.record()
    torch.cuda.synchronize()
    ms = s.elapsed_time(e) / reps
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    lib.gemb_check_device_status()
    flops = 2.0 * tokens * 3 * inter * hidden
    return {"metric": "tensor-parallel MLP tokens/s", "ranks": world, "tokens": tokens, "ms": ms,
            "tokens_per_s": tokens / ms * 1e3, "tflops_aggregate": flops / ms / 1e9,
            "reduction": {"peer": "reduce-scatter + all-gather kernels over peer memory, flag barriers",
                          "nccl": "NCCL all-reduce of the fp32 partials"}[mlp.reduce] if world > 1 else "none",
            "partial_bytes_per_rank": tokens * hidden * 4 if world > 1 else 0}


def bench_moe_ep(lib, dev, world, rank, layers=30, phases=((16384, "prefill"), (64, "decode"))):
    """Expert-parallel MoE stack: `layers` distinct 26B-A4B-like layers, experts split evenly over
    the ranks, tokens data-sharded; dispatch and combine by the library's pull kernels over peer
    memory (NCCL all-to-all if no peer mapping can be had).  Collective: every rank calls it;
    returns the summary on every rank (times are the max over ranks)."""
    import torch
    import torch.distributed as dist
    from gem16_b200.ep import EpMoeLayer, EpPullMoeLayer
    from gem16_b200.moe import MoeLayer, synthetic_weights
    experts = 128
    e_local = experts // world
    rng = (rank * e_local, (rank + 1) * e_local)
    weights = [synthetic_weights(dev, SEED + 4000 + l, expert_range=rng if world > 1 else None, placement_ranks=world)
               for l in range(layers)]
    out = {"metric": "MoE stack tokens/s", "layers": layers, "ranks": world, "experts_per_rank": e_local, "phases": {}}
    for tokens, name in phases:
        t_local = tokens // world
        gen = torch.Generator(device=dev)
        gen.manual_seed(SEED + 4100)
        x_all = torch.randn((tokens, 2816), device=dev, generator=gen).to(torch.bfloat16)
        ga = float(2688.0 / x_all.float().abs().max().item())
        x = x_all[rank * t_local:(rank + 1) * t_local].contiguous().view(torch.int16)
        if world > 1:
            try:
                shared_bufs = EpPullMoeLayer(weights[0], t_local, 8, ga, 336.0, 336.0)
                out["exchange"] = "pull kernels over peer memory (" + shared_bufs.send.how + ")"
            except Exception as exc:
                shared_bufs = EpMoeLayer(weights[0], t_local, 8, ga, 336.0, 336.0)
                out["exchange"] = f"NCCL all-to-all ({type(exc).__name__}: {exc})"[:300]
            def run():
                for w in weights:
                    shared_bufs.w = w
                    shared_bufs.local.w = w
                    shared_bufs.forward(x)
        else:
            buf = MoeLayer(weights[0], tokens, 8, ga, 336.0, 336.0)
            def run():
                st = torch.cuda.current_stream()
                for w in weights:
                    buf.w = w
                    buf.forward(x, st)
        for _ in range(2):
            run()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        # The launch sequence is fixed (nothing is read back to the host), so the whole stack --
        # the two NCCL collectives per layer included -- replays as one CUDA graph.  All ranks
        # agree on whether the capture worked; otherwise the stack runs eagerly.
        step, mode, graph = run, "eager", None
        if "NCCL all-to-all" not in out.get("exchange", ""):
            st = torch.cuda.Stream(device=dev)
            ok = 1
            try:
                with torch.cuda.stream(st):
                    run()
                    st.synchronize()
                    graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(graph, stream=st):
                        run()
                    graph.replay()
                    st.synchronize()
            except Exception:
                ok = 0
            if world > 1:
                okt = torch.tensor([ok], device=dev)
                dist.all_reduce(okt, op=dist.ReduceOp.MIN)
                ok = int(okt.item())
            if ok:
                step, mode = graph.replay, "cuda graph"
        out.setdefault("launch", {})[name] = mode
        for _ in range(2):
            step()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 3
        s.record()
        for _ in range(reps):
            step()
        e.record()
        torch.cuda.synchronize()
        ms = s.elapsed_time(e) / reps
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        lib.gemb_check_device_status()
        out["phases"][name] = {"tokens": tokens, "ms_per_stack": ms, "tokens_per_s": tokens / ms * 1e3,
                               "us_per_layer": ms * 1e3 / layers}
        del x_all, step, graph
        if world > 1:
            del shared_bufs
        else:
            del buf
        torch.cuda.empty_cache()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="decode_gemv", choices=["decode_gemv"])
    ap.add_argument("--decode-path", default="split", choices=["fused", "split"],
                    help="decode GEMV set: activation quantisation fused into the GEMV, or quantizer + GEMV launches")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-other-workloads", action="store_true")
    ap.add_argument("--layers", type=int, default=LAYERS,
                    help="decode layers held on the device (48 = the benchmark; fewer for a small profiler capture)")
    ap.add_argument("--only", default=None, choices=["nvfp4_linear", "moe_layer", "prefill_gemm", "prefill_stack", "output_head", "verifier_gemv"],
                    help="run just one secondary workload on one GPU and print its JSON (profiling aid)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
        return
    if args.only:
        import torch
        from gem16_b200 import load
        dev = torch.device("cuda", 0)
        torch.cuda.set_device(dev)
        fn = {"nvfp4_linear": bench_nvfp4_linear, "moe_layer": bench_moe_layer, "prefill_gemm": bench_prefill_gemm,
              "prefill_stack": bench_prefill_stack, "output_head": bench_output_head,
              "verifier_gemv": bench_verifier_gemv}[args.only]
        print(json.dumps(fn(load(), dev)), flush=True)
        return
    run_decode_gemv(args)


if __name__ == "__main__":
    main()
