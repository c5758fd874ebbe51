#!/usr/bin/env python
"""Benchmark of the quantized-contraction hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    torchrun --nproc-per-node N bench.py --gpus N ...        (one rank per GPU)

One JSON line on stdout (rank 0).  The headline workload is the expert-parallel MoE stack, the one
of the path's three metrics that is defined at 1, 2, 4 and 8 GPUs:

  moe_ep_stack_prefill   30 distinct 26B-A4B-like MoE layers (hidden 2816, 128 experts x 704, top-8,
                shared FFN 2112, NVFP4 W4A4) over a 16,384-token batch.  Experts are split evenly over
                the ranks, tokens are data-sharded (16,384 / N per rank), the router is replicated;
                dispatch and combine run over NVLink peer memory inside the library's layer call.
                A step is one pass of the batch through all 30 layers, replayed as one CUDA graph.
                The total work is fixed as N grows (strong scaling).  Metric: tokens/s.

`value` is measured with the tokens resident in HBM; `e2e` copies each rank's tokens from pinned
host memory and the bf16 result back inside the timed region, every step, on a copy stream: the next
step's upload and the previous step's download run under the current step's layers, as a serving loop
would overlap them, and the region closes only when the last result is in host memory.  The 64-token decode batch through
the same stack is reported beside it, and the other workloads of the path (decode GEMV set, the
single NVFP4 linear, the 4,096-token MoE layer, the dense prefill projections, output head,
verifier GEMV, tensor-parallel MLP) under "other_workloads", each with its own roofline and, for
the three named metrics, CPU baseline and end-to-end figures.

Every rank feeds every layer the same seeded N(0,1) tokens (the layers differ in their weights):
chaining the layers without the norms and residuals that sit between them in the model would let the
activations drift off the quantisers' static scales and the routing collapse.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# Exactly one line goes to stdout, the result.  Libraries that print to file descriptor 1 (NCCL's
# version banner, for one) are sent to stderr instead: descriptor 1 is pointed at descriptor 2 and
# the result is written to a saved copy of the original.
_RESULT_FD = os.dup(1)
os.dup2(2, 1)


def emit(line: dict) -> None:
    os.write(_RESULT_FD, (json.dumps(line) + "\n").encode())

DECODE_SHAPES = [("gate_up", 30720, 3840), ("down", 3840, 15360), ("qkv", 8192, 3840), ("o", 3840, 4096)]
LAYERS = 48            # decode GEMV set
MOE_LAYERS = 30
MOE = dict(hidden=2816, experts=128, inter=704, shared_inter=2112, topk=8)
SEED = 20261125
FP4_NOMINAL_TFLOPS = 9000.0      # dense NVFP4, vendor figure; no measured FP4 peak exists on this pool
FP8_NOMINAL_TFLOPS = 4500.0


def decode_bytes_per_layer() -> int:
    """Algorithmic bytes of one decode layer: weights + fp32-equivalent scales + bf16 x + bf16 y."""
    total = 0
    for _, rows, k in DECODE_SHAPES:
        total += rows * k + rows * 4 + k * 2 + rows * 2
    return total


def moe_layer_flops(tokens: int) -> dict:
    h, e, i, s, k = MOE["hidden"], MOE["experts"], MOE["inter"], MOE["shared_inter"], MOE["topk"]
    return {"router": 2.0 * tokens * e * h, "experts": tokens * k * 2.0 * 3 * i * h, "shared": tokens * 2.0 * 3 * s * h}


def moe_layer_weight_bytes() -> float:
    h, e, i, s = MOE["hidden"], MOE["experts"], MOE["inter"], MOE["shared_inter"]
    return e * 3 * i * h * 0.5625 + 3 * s * h * 0.5625 + e * h * 4


def measured_peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d.get("bf16_tflops", 1590.0)),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", 1400.0)), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def profile_traffic(name: str):
    """dram__bytes_read.sum + dram__bytes_write.sum per launch of a kernel, as recorded in the kept ncu
    summary of that kernel (a line `traffic_bytes_per_launch: <n>` together with the algorithmic bytes
    or flops of the captured launch).  None when no summary holds the figure."""
    path = os.path.join(ROOT, "profiles", name)
    out = {}
    try:
        with open(path) as f:
            for line in f:
                for key in ("traffic_bytes_per_launch", "captured_units_per_launch"):
                    if line.strip().startswith(key + ":"):
                        out[key] = float(line.split(":", 1)[1].split()[0].replace(",", ""))
    except OSError:
        return None
    return out or None


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""

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
        return self

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
# CPU baselines / reference arm: the reference's own CPU numeric functions on bounded samples
# --------------------------------------------------------------------------------------------
def cpu_oracles(use_ref: bool):
    from oracle import Oracle, default_threads, ref_available
    kind = "reference" if use_ref and ref_available() else "port"
    return Oracle(ref=(kind == "reference")), Oracle(), default_threads(), kind


def cpu_decode_sample(steps: int, warmup: int, use_ref: bool):
    """One decode layer (four FP8 GEMVs incl. the per-token quantisation) on the host cores with gem16's
    src/numeric/fp8.cpp functions.  Returns (GB/s, seconds per layer, cores, kind)."""
    import numpy as np
    o, port, threads, kind = cpu_oracles(use_ref)
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


def cpu_linear_sample(use_ref: bool, tokens: int = 8):
    """`tokens` rows of the single NVFP4 linear (K = 3840, 15,360 output rows): gem16's QuantizeActivation
    and ReferenceDotProduct (src/numeric/nvfp4.cpp:113-201).  Returns (TFLOP/s, seconds, cores, kind)."""
    import numpy as np
    o, port, threads, kind = cpu_oracles(use_ref)
    rng = np.random.default_rng(SEED + 1)
    n, k = 15360, 3840
    wp = rng.integers(0, 256, size=(n, k // 2), dtype=np.uint8)
    ws = rng.integers(0x30, 0x48, size=(n, k // 16), dtype=np.uint8)
    x = port.from_bf16(port.to_bf16(rng.standard_normal((tokens, k)).astype(np.float32)))
    t0 = time.perf_counter()
    xp, xs = o.nvfp4_quantize(x, 600.0, threads=threads)
    o.nvfp4_matmul(xp, xs, wp, ws, 600.0, 9000.0, threads=threads)
    dt = time.perf_counter() - t0
    return 2.0 * tokens * n * k / dt / 1e12, dt, threads, kind


_CPU_MOE_CACHE = {}


def cpu_moe_layer_sample(use_ref: bool, tokens: int = 64, fresh: bool = False):
    """Cached wrapper (the own arm reports the same sample under two workloads)."""
    key = (use_ref, tokens)
    if fresh or key not in _CPU_MOE_CACHE:
        _CPU_MOE_CACHE[key] = _cpu_moe_layer_sample(use_ref, tokens)
    return _CPU_MOE_CACHE[key]


def _cpu_moe_layer_sample(use_ref: bool, tokens: int = 64):
    """One MoE layer on `tokens` tokens on the host cores: router, top-8, stable permutation and combine
    through the CPU restatement of the specifications (gem16 has no MoE code), every expert and shared
    projection through gem16's own QuantizeActivation / ReferenceDotProduct.  One random expert matrix
    stands in for all 128 (only the time is wanted).  Returns (seconds per layer, cores, kind)."""
    import numpy as np
    o, port, threads, kind = cpu_oracles(use_ref)
    rng = np.random.default_rng(SEED + 3)
    h, e, i, s, k = MOE["hidden"], MOE["experts"], MOE["inter"], MOE["shared_inter"], MOE["topk"]

    def rand_w(rows, kk):
        return (rng.integers(0, 256, size=(rows, kk // 2), dtype=np.uint8),
                rng.integers(0x30, 0x48, size=(rows, kk // 16), dtype=np.uint8))

    gu, dn, sgu, sdn = rand_w(2 * i, h), rand_w(h, i), rand_w(2 * s, h), rand_w(h, s)
    router_w = (rng.standard_normal((e, h)) * 0.02).astype(np.float32)
    rank = rng.permutation(e) + 1
    bias = (-1.1 * np.log(rank)).astype(np.float32)
    xb = port.to_bf16(rng.standard_normal((tokens, h)).astype(np.float32))
    x = port.from_bf16(xb)

    def ffn(xq, xs, wgu, wdn, inter):
        gate_up = port.from_bf16(port.to_bf16(o.nvfp4_matmul(xq, xs, wgu[0], wgu[1], 600.0, 9000.0, threads=threads).astype(np.float32)))
        prod = port.gated_gelu(gate_up[:, :inter], gate_up[:, inter:])
        pq, ps = o.nvfp4_quantize(prod, 336.0, threads=threads)
        return port.to_bf16(o.nvfp4_matmul(pq, ps, wdn[0], wdn[1], 336.0, 9000.0, threads=threads).astype(np.float32))

    t0 = time.perf_counter()
    logits = port.moe_router_logits(xb, router_w, bias, threads=threads)
    ids, weights = port.moe_route(logits, k)
    counts, offsets, perm = port.moe_permute(ids, e)
    xq, xs = o.nvfp4_quantize(x, 600.0, threads=threads)
    y = np.zeros((tokens * k, h), np.uint16)
    for ex in range(e):
        sel = perm[offsets[ex]:offsets[ex + 1]]
        if sel.size:
            y[sel] = ffn(xq[sel // k], xs[sel // k], gu, dn, i)
    shared = ffn(xq, xs, sgu, sdn, s)
    port.moe_combine(y.reshape(tokens, k, h), weights, shared)
    return time.perf_counter() - t0, threads, kind


def run_reference_arm(args):
    """The reference's CPU numeric path on this box's host cores, for the headline workload: each step
    is one MoE layer on a 64-token sample; tokens/s of the whole 30-layer stack is that rate / 30."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    tokens = int(os.environ.get("GEMB_BENCH_REFERENCE_TOKENS", "64"))   # the CPU test suite shrinks the sample
    steps = max(1, min(args.steps, 5))
    times = []
    for _ in range(min(args.warmup, 1) + steps):
        dt, cores, kind = cpu_moe_layer_sample(use_ref=True, tokens=tokens, fresh=True)
        times.append(dt)
    dt = statistics.median(times[-steps:])
    value = tokens / (dt * MOE_LAYERS)
    sample = (f"{tokens}-token sample of ONE of the {MOE_LAYERS} layers per step ({dt:.2f} s on {cores} host threads); "
              f"tokens/s of the stack = sample rate / {MOE_LAYERS} (extrapolated: CPU time is linear in tokens and layers)")
    line = {
        "impl": "reference", "metric": "MoE stack tokens/s", "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": min(args.warmup, 1), "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "nvfp4 (binary64 accumulate on the CPU)", "data": "synthetic",
        "config": moe_config(args.gpus),
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cores, "kind": kind, "sample": sample,
                         "note": "expert and shared projections: gem16 src/numeric/nvfp4.cpp; router / permutation / combine: "
                                 "CPU restatement of gem16's MoE specifications (gem16 has no MoE code)"},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    emit(line)


def moe_config(world: int) -> dict:
    return {"workload": "moe_ep_stack_prefill", "layers": MOE_LAYERS, "tokens": 16384, **MOE,
            "format": "NVFP4 W4A4, E4M3 block scales per 16, fp32 global divisors",
            "parallelism": f"ep{world}" if world > 1 else "single GPU",
            "l2": "30 distinct layers of expert weights, 12.8 GB per pass >> 126 MB L2",
            "inputs": "every layer reads the same seeded N(0,1) bf16 tokens; router bias Zipf(1.1)"}


# --------------------------------------------------------------------------------------------
# headline: the expert-parallel MoE stack
# --------------------------------------------------------------------------------------------
STAGE_BITS = {"route": 1, "pack": 2, "gate_up": 4, "gelu": 8, "down": 16, "combine": 32, "shared": 64, "exchange": 128}


class Dist:
    """Rank plumbing: NCCL process group when launched with torchrun, trivial otherwise."""

    def __init__(self):
        import torch
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        if self.world > 1:
            import torch.distributed as dist
            dist.init_process_group("nccl", device_id=self.dev)

    def barrier(self):
        import torch
        torch.cuda.synchronize(self.dev)
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize(self.dev)

    def max(self, value: float) -> float:
        if self.world == 1:
            return value
        import torch
        import torch.distributed as dist
        t = torch.tensor([value], device=self.dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def all_true(self, flag: bool) -> bool:
        if self.world == 1:
            return flag
        import torch
        import torch.distributed as dist
        t = torch.tensor([1 if flag else 0], device=self.dev)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        return bool(t.item())

    def close(self):
        if self.world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()


def timed_region(d: Dist, stream, fn, steps: int, tail=None) -> float:
    """Seconds for exactly `steps` calls of fn: CUDA events on the launching stream, a barrier and a
    device synchronise on both sides, the maximum over ranks.  `tail` (optional) is enqueued behind the
    last step and before the closing event: it makes the stream wait for work the steps left on other streams."""
    import torch
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    d.barrier()
    start.record(stream)
    for _ in range(steps):
        fn()
    if tail is not None:
        tail()
    end.record(stream)
    d.barrier()
    return d.max(start.elapsed_time(end) / 1e3)


def repeated_regions(d: Dist, stream, fn, steps: int, min_seconds: float = 0.5, max_regions: int = 9, tail=None):
    """Runs the K-step region until at least min_seconds of device time have been measured (at most
    max_regions times) and returns (median seconds per region, all samples)."""
    samples = []
    while len(samples) < 1 or (sum(samples) < min_seconds and len(samples) < max_regions):
        samples.append(timed_region(d, stream, fn, steps, tail))
    return statistics.median(samples), samples


def capture(stream, enqueue):
    """enqueue() once eagerly, then captured (twice: a graph with a forked side stream instantiated right
    after the eager pass has replayed measurably slower here than the same capture taken once more)."""
    import torch
    with torch.cuda.stream(stream):
        enqueue()
        stream.synchronize()
        for _ in range(2):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                enqueue()
            g.replay()
            stream.synchronize()
    return g


def run_moe_stack(args):
    import torch
    from gem16_b200 import load
    from gem16_b200.ep import EpLayer
    from gem16_b200.moe import MoeLayer, synthetic_weights

    d = Dist()
    dev, world, rank = d.dev, d.world, d.rank
    lib = load()
    lib.gemb_device_check()
    if args.ep_shared_sms is not None:
        lib.gemb_set_tuning(9, args.ep_shared_sms)
    if args.ep_split_sms is not None:
        lib.gemb_set_tuning(10, args.ep_split_sms)
    layers = args.moe_layers
    e_local = MOE["experts"] // world
    own = (rank * e_local, (rank + 1) * e_local)
    weights = [synthetic_weights(dev, SEED + 4000 + l, expert_range=own if world > 1 else None, placement_ranks=world)
               for l in range(layers)]
    topk, h = MOE["topk"], MOE["hidden"]
    phases = {}
    stream = torch.cuda.Stream(device=dev)
    for name, tokens in (("prefill", 16384), ("decode", 64)):
        t_local = tokens // world
        gen = torch.Generator(device=dev)
        gen.manual_seed(SEED + 4100)
        x_all = torch.randn((tokens, h), device=dev, generator=gen).to(torch.bfloat16)
        ga = float(2688.0 / x_all.float().abs().max().item())
        x_dev = x_all[rank * t_local:(rank + 1) * t_local].contiguous().view(torch.int16)
        x_host = x_dev.cpu().pin_memory()
        out_host = torch.empty((t_local, h), dtype=torch.int16).pin_memory()
        if world > 1:
            obj = EpLayer(weights[0], t_local, topk, ga, 336.0, 336.0, fused=args.fused)
        else:
            obj = MoeLayer(weights[0], tokens, topk, ga, 336.0, 336.0, stages=False)
            obj.fused = args.fused

        def enqueue():
            for w in weights:
                obj.w = w
                if world > 1:
                    obj.forward(x_dev)
                else:
                    obj.forward(x_dev, torch.cuda.current_stream())

        graph = capture(stream, enqueue)

        # End to end, as a serving loop would run it: every step's tokens come from pinned host memory and every
        # step's result goes back to it, on a copy stream, so that step i + 1's upload and step i - 1's download
        # run under step i's layers.  Staging buffers on the device decouple the copies from the graph's fixed
        # input and output: the compute stream takes the staged tokens (device-to-device) before its layers and
        # leaves the result in a staging buffer behind them.
        copy_stream = torch.cuda.Stream(device=dev)
        x_stage, out_stage = torch.empty_like(x_dev), torch.empty_like(obj.out)
        ev_h2d, ev_taken, ev_out, ev_d2h = (torch.cuda.Event() for _ in range(4))

        def upload():
            with torch.cuda.stream(copy_stream):
                copy_stream.wait_event(ev_taken)          # the previous tokens have left the staging buffer
                x_stage.copy_(x_host, non_blocking=True)
                ev_h2d.record(copy_stream)

        def step_e2e():
            stream.wait_event(ev_h2d)                     # this step's tokens have arrived
            x_dev.copy_(x_stage, non_blocking=True)
            ev_taken.record(stream)
            upload()                                      # the next step's tokens, under this step's layers
            graph.replay()
            stream.wait_event(ev_d2h)                     # the previous result has left its staging buffer
            out_stage.copy_(obj.out, non_blocking=True)
            ev_out.record(stream)
            with torch.cuda.stream(copy_stream):
                copy_stream.wait_event(ev_out)
                out_host.copy_(out_stage, non_blocking=True)
                ev_d2h.record(copy_stream)

        def step_e2e_serial():
            """The same step with nothing overlapped: upload, layers, download, host synchronise."""
            x_dev.copy_(x_host, non_blocking=True)
            graph.replay()
            out_host.copy_(obj.out, non_blocking=True)
            stream.synchronize()

        def e2e_tail():
            stream.wait_event(ev_d2h)                     # the last result is in host memory
            stream.wait_event(ev_h2d)                     # and the look-ahead upload has ended

        with torch.cuda.stream(stream):
            for _ in range(max(args.warmup, 3)):
                graph.replay()
            sampler = ClockSampler(d.local).start() if rank == 0 else None
            secs, samples = repeated_regions(d, stream, graph.replay, args.steps)
            clocks = sampler.stop() if sampler else None
            ev_taken.record(stream)
            ev_d2h.record(stream)
            upload()
            for _ in range(2):
                step_e2e()
            secs_e2e, _ = repeated_regions(d, stream, step_e2e, args.steps, tail=e2e_tail)
            stream.synchronize()
            copy_stream.synchronize()
            secs_e2e_serial = timed_region(d, stream, step_e2e_serial, args.steps)
            lib.gemb_check_device_status()
            # Stage by stage: the same graph with one stage of the layer call enabled at a time, on the
            # workspace the full pass left behind (each layer's own weights, the last layer's plan).
            stage_us = {}
            counts_total = int(obj.counts.sum().item()) if world == 1 else int(obj.counts_all[:, own[0]:own[1]].sum().item())
            if not args.no_stage_times:
                for sname, bit in STAGE_BITS.items():
                    if sname == "gelu" and args.fused:
                        continue
                    if sname == "exchange" and world == 1:
                        continue
                    lib.gemb_set_tuning(7, bit)
                    try:
                        g = capture(stream, enqueue)
                        for _ in range(2):
                            g.replay()
                        t = timed_region(d, stream, g.replay, 5) / 5 / layers
                        stage_us[sname] = t * 1e6
                    finally:
                        lib.gemb_set_tuning(7, 0)
                    del g
                lib.gemb_check_device_status()
        phases[name] = {"tokens": tokens, "tokens_per_rank": t_local, "secs_per_step": secs / args.steps,
                        "region_samples_s": samples, "secs_per_step_e2e": secs_e2e / args.steps, "secs_per_step_e2e_serial": secs_e2e_serial / args.steps, "clocks": clocks,
                        "stage_us_per_layer": stage_us, "assignments_on_rank0_last_layer": counts_total,
                        "h2d_bytes": x_host.numel() * 2 * world, "d2h_bytes": out_host.numel() * 2 * world,
                        "exchange": ("peer memory, " + obj.send.how) if world > 1 else "none"}
        del graph, obj, x_all
        torch.cuda.empty_cache()

    # Bit-exactness of the expert-parallel layer against the single-GPU layer, on every rank, outside
    # the timed regions: at 96 tokens per rank (the small-batch launch sequence) and at the benchmark's
    # prefill size (the large-batch sequence that was timed above).
    parity = None
    if world > 1:
        full = synthetic_weights(dev, SEED + 4000, placement_ranks=world)
        checks = []
        for t_local in (96, 16384 // world):
            gen = torch.Generator(device=dev)
            gen.manual_seed(SEED + 4200 + t_local)
            x_all = torch.randn((t_local * world, h), device=dev, generator=gen).to(torch.bfloat16).view(torch.int16)
            sl = slice(rank * t_local, (rank + 1) * t_local)
            ref = MoeLayer(full, t_local * world, topk, 600.0, 336.0, 336.0, stages=False)
            ref.fused = args.fused
            want = ref.forward(x_all).clone()
            ref_local = MoeLayer(full, t_local, topk, 600.0, 336.0, 336.0, stages=False)
            ref_local.fused = args.fused
            ref_local.forward(x_all[sl].contiguous())
            ep = EpLayer(weights[0], t_local, topk, 600.0, 336.0, 336.0, fused=args.fused)
            for _ in range(2):
                got = ep.forward(x_all[sl].contiguous())
            torch.cuda.synchronize()
            lib.gemb_check_device_status()
            routing = (torch.equal(ep.ids, ref.ids[sl]) and torch.equal(ep.weights, ref.weights[sl])
                       and torch.equal(ep.counts_all.sum(0).to(torch.int32), ref.counts)
                       and torch.equal(ep.counts, ref_local.counts) and torch.equal(ep.perm, ref_local.perm))
            checks.append({"tokens_per_rank": t_local, "ids_counts_perm_bit_exact": d.all_true(bool(routing)),
                           "output_bit_exact": d.all_true(bool(torch.equal(got, want[sl])))})
            del ref, ref_local, ep, x_all, want, got
            torch.cuda.empty_cache()
        parity = {"ranks": world, "tokens_per_rank": checks[0]["tokens_per_rank"],
                  "ids_counts_perm_bit_exact": checks[0]["ids_counts_perm_bit_exact"],
                  "output_bit_exact": checks[0]["output_bit_exact"], "prefill_size": checks[1]}
        del full
        torch.cuda.empty_cache()
    del weights
    torch.cuda.empty_cache()
    return d, lib, phases, parity


def moe_headline(args):
    d, lib, phases, parity = run_moe_stack(args)
    import torch
    world, rank, dev = d.world, d.rank, d.dev
    layers = args.moe_layers
    others = {}
    if not args.no_other_workloads:
        if world > 1:
            try:
                others["tp_mlp"] = bench_tp_mlp(lib, dev, world, rank)
            except Exception as exc:
                others["tp_mlp"] = {"error": f"{type(exc).__name__}: {exc}"}
        elif rank == 0:
            for name, fn in (("decode_gemv", bench_decode_gemv), ("nvfp4_linear", bench_nvfp4_linear), ("moe_layer", bench_moe_layer),
                             ("prefill_gemm", bench_prefill_gemm), ("prefill_stack", bench_prefill_stack),
                             ("output_head", bench_output_head), ("verifier_gemv", bench_verifier_gemv)):
                try:
                    others[name] = fn(lib, dev, args)
                except Exception as exc:  # a secondary workload must not take the headline line down
                    others[name] = {"error": f"{type(exc).__name__}: {exc}"}
    if rank != 0:
        d.close()
        return
    pre, dec = phases["prefill"], phases["decode"]
    tokens = pre["tokens"]
    value = tokens / pre["secs_per_step"]
    flops = moe_layer_flops(tokens)
    peaks = measured_peaks()
    # Roofline of the dominant kernel, the grouped gate/up GEMM of rank 0: algorithmic flops of one launch
    # (the rank's real assignments x 2 x 1408 x 2816) over its average duration in a graph that launches
    # only that kernel for every layer.
    gate_us = pre["stage_us_per_layer"].get("gate_up")
    roof = None
    if gate_us:
        launch_flops = pre["assignments_on_rank0_last_layer"] * 2.0 * 2 * MOE["inter"] * MOE["hidden"]
        achieved = launch_flops / (gate_us * 1e-6) / 1e12
        prof = profile_traffic("gemm_kernel_grouped_gate_up.md")
        traffic = None
        if prof and prof.get("captured_units_per_launch"):
            traffic = prof["traffic_bytes_per_launch"] * pre["assignments_on_rank0_last_layer"] / prof["captured_units_per_launch"]
        roof = {"bound": "tensor", "kernel": "gemm_kernel<nvfp4, grouped 128x256> gate/up" + (" + GELU requantising epilogue" if args.fused else ""),
                "achieved": achieved, "peak": FP4_NOMINAL_TFLOPS, "unit": "TFLOP/s", "frac": achieved / FP4_NOMINAL_TFLOPS,
                "peak_source": "nominal dense NVFP4 (9 PFLOP/s): no measured FP4 peak exists for this pool",
                "frac_of_4x_measured_bf16": achieved / (4 * peaks["bf16_tflops"]),
                "avg_launch_us": gate_us, "flops_per_launch": launch_flops,
                "time_x_sm_mhz": gate_us * (pre["clocks"]["sm_mhz"] or 0) if pre["clocks"] else None,
                "traffic": traffic, "traffic_unit": "dram bytes per launch, scaled from the kept ncu capture by assignments",
                "per_rank_bound_us_per_layer": {
                    "tensor_at_nominal": sum(flops.values()) / world / (FP4_NOMINAL_TFLOPS * 1e12) * 1e6,
                    "weights_over_hbm": moe_layer_weight_bytes() / world / (peaks["hbm_gbs"] * 1e9) * 1e6,
                    "nvlink_combine": (tokens / world) * MOE["topk"] * (world - 1) / world * MOE["hidden"] * 2 / 770e9 * 1e6}}
    launches_per_layer = (11 if args.fused else 12) + (3 if world > 1 else 0)
    line = {
        "metric": "MoE stack tokens/s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": pre["secs_per_step"] * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "nvfp4 (W4A4, fp32 accumulate)", "data": "synthetic",
        "config": dict(moe_config(world), layers=layers, exchange=pre["exchange"], fused_gelu_epilogue=bool(args.fused),
                       timing=f"median of {len(pre['region_samples_s'])} regions of {args.steps} steps"),
        "e2e": {"value": tokens / pre["secs_per_step_e2e"], "unit": "tokens/s", "h2d_bytes_per_step": pre["h2d_bytes"],
                "d2h_bytes_per_step": pre["d2h_bytes"],
                "how": "every step uploads its tokens from pinned host memory and downloads its result; the copies run on a "
                       "second stream under the neighbouring steps' layers; the region ends when the last result is in host memory",
                "not_overlapped": tokens / pre["secs_per_step_e2e_serial"]},
        "gpu_launches": launches_per_layer * layers * args.steps,
        "clocks": pre["clocks"],
        "roofline": roof,
        "us_per_layer": pre["secs_per_step"] / layers * 1e6,
        "stage_us_per_layer": pre["stage_us_per_layer"],
        "decode_phase": {"tokens": 64, "value": 64 / dec["secs_per_step"], "unit": "tokens/s",
                         "us_per_layer": dec["secs_per_step"] / layers * 1e6,
                         "e2e": 64 / dec["secs_per_step_e2e"], "stage_us_per_layer": dec["stage_us_per_layer"],
                         "clocks": dec["clocks"]},
    }
    if parity is not None:
        line["ep_parity"] = parity
    if others:
        line["other_workloads"] = others
    if world == 1 and not args.no_cpu_baseline:
        dt, cores, kind = cpu_moe_layer_sample(use_ref=True, tokens=64)
        line["cpu_baseline"] = {"value": 64 / (dt * layers), "unit": "tokens/s", "cores": cores, "kind": kind,
                                "sample": f"64 tokens through one of the {layers} layers: {dt:.2f} s on {cores} host threads; "
                                          f"stack rate extrapolated as sample rate / {layers}"}
    emit(line)
    d.close()


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


def bench_nvfp4_linear(lib, dev, args=None):
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

    reps = 3000      # 8 linears per replay: about half a second of device time
    t_gemm, clocks = sampled(lambda: graph_time(gemm_only, copies, reps=reps) / copies, dev.index or 0)
    t_both = graph_time(quant_and_gemm, 2 * copies, reps=reps // 2) / copies
    # end to end: bf16 activations from pinned host memory, quantiser + GEMM, bf16 result back
    x_host = x.view(torch.int16).cpu().pin_memory()
    y_host = torch.empty((m, n), dtype=torch.int16).pin_memory()
    st = torch.cuda.Stream(device=dev)
    xi = x.view(torch.int16)
    with torch.cuda.stream(st):
        def e2e_step(i):
            wq, wsc, gw = ws[i % copies]
            xi.copy_(x_host, non_blocking=True)
            lib.gemb_nvfp4_quantize(xi, 1, xq, xs, m, k, ga, 1, 0, st)
            lib.gemb_nvfp4_gemm_bf16(xq, xs, wq, wsc, out, m, n, k, ga, gw, st)
            y_host.copy_(out, non_blocking=True)
            st.synchronize()
        for i in range(3):
            e2e_step(i)
        t0 = time.perf_counter()
        for i in range(40):
            e2e_step(i)
        t_e2e = (time.perf_counter() - t0) / 40
    lib.gemb_check_device_status()
    flops = 2.0 * m * n * k
    peaks = measured_peaks()
    res = {"metric": "NVFP4 GEMM TFLOP/s", "workload": "nvfp4_linear 512x15360x3840 (W4A4)",
           "value": flops / t_gemm / 1e12, "unit": "TFLOP/s", "us_per_linear": t_gemm * 1e6, "dtype": "nvfp4 (W4A4, fp32 accumulate)",
           "with_activation_quantizer": {"value": flops / t_both / 1e12, "us_per_linear": t_both * 1e6},
           "e2e": {"value": flops / t_e2e / 1e12, "unit": "TFLOP/s", "us_per_linear": t_e2e * 1e6,
                   "h2d_bytes_per_step": m * k * 2, "d2h_bytes_per_step": m * n * 2},
           "clocks": clocks, "timed_region_s": t_gemm * copies * reps,
           "roofline": {"bound": "tensor", "kernel": "gemm_kernel<nvfp4, 256x256 on CTA pairs>", "achieved": flops / t_gemm / 1e12,
                        "peak": FP4_NOMINAL_TFLOPS, "unit": "TFLOP/s", "frac": flops / t_gemm / 1e12 / FP4_NOMINAL_TFLOPS,
                        "peak_source": "nominal dense NVFP4 (9 PFLOP/s): no measured FP4 peak exists for this pool",
                        "frac_of_4x_measured_bf16": flops / t_gemm / 1e12 / (4 * peaks["bf16_tflops"]),
                        "time_x_sm_mhz": t_gemm * 1e6 * (clocks["sm_mhz"] or 0)},
           "l2": f"{copies} distinct weight sets in rotation, {copies * (n * k // 2 + n * k // 16) / 1e6:.0f} MB > 126 MB L2"}
    if args is None or not args.no_cpu_baseline:
        tf, dt, cores, kind = cpu_linear_sample(use_ref=True, tokens=8)
        res["cpu_baseline"] = {"value": tf, "unit": "TFLOP/s", "cores": cores, "kind": kind,
                               "sample": f"8 of the 512 tokens x all 15,360 rows (gem16 QuantizeActivation + ReferenceDotProduct): {dt:.2f} s on {cores} host threads"}
    return res


def bench_prefill_gemm(lib, dev, args=None):
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


def bench_prefill_stack(lib, dev, args=None, layers=48, tokens=16384):
    """Dense 12B-like prefill linear stack: per layer FP8 QKV and O projections and the NVFP4 gated
    MLP (gate/up GEMM + GELU + requantisation as one kernel on weights packed once at load time),
    every activation quantiser inside the timed region (attention itself is replaced by a seeded bf16
    tensor: it is not part of this path)."""
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

    def fp4_w(n, k, interleaved=True):
        w = torch.randn((n, k), device=dev, generator=gen) * 0.02
        g = float(2688.0 / w.abs().max().item())
        q = torch.empty((n, k // 2), dtype=torch.uint8, device=dev)
        s = (torch.zeros((c.gemb_interleaved_scale_bytes(n, k),), dtype=torch.uint8, device=dev) if interleaved
             else torch.empty((n, k // 16), dtype=torch.uint8, device=dev))
        lib.gemb_nvfp4_quantize(w, 0, q, s, n, k, g, 1 if interleaved else 0, 0, None)
        return q, s, g

    def gate_up_w():
        (gq, gs, gg), (uq, us, gu) = fp4_w(inter, h, False), fp4_w(inter, h, False)
        fq = torch.empty((2 * inter, h // 2), dtype=torch.uint8, device=dev)
        fs = torch.zeros((c.gemb_interleaved_scale_bytes(2 * inter, h),), dtype=torch.uint8, device=dev)
        lib.gemb_nvfp4_pack_gate_up(gq, gs, uq, us, fq, fs, inter, h, None)
        return fq, fs, gg, gu

    weights = [(fp8_w(qkv, h), fp8_w(h, ao), gate_up_w(), fp4_w(h, inter)) for _ in range(layers)]
    x = torch.randn((tokens, h), device=dev, generator=gen).to(torch.bfloat16).view(torch.int16)
    attn = torch.randn((tokens, ao), device=dev, generator=gen).to(torch.bfloat16).view(torch.int16)
    u8 = dict(dtype=torch.uint8, device=dev)
    xq, xs = torch.empty((tokens, h), **u8), torch.empty((tokens,), device=dev)
    aq, as_ = torch.empty((tokens, ao), **u8), torch.empty((tokens,), device=dev)
    y_qkv = torch.empty((tokens, qkv), dtype=torch.int16, device=dev)
    y_o = torch.empty((tokens, h), dtype=torch.int16, device=dev)
    oq = torch.empty((tokens, h // 2), **u8)
    os_ = torch.zeros((c.gemb_interleaved_scale_bytes(tokens, h),), **u8)
    pq = torch.empty((tokens, inter // 2), **u8)
    ps = torch.zeros((c.gemb_interleaved_scale_bytes(tokens, inter),), **u8)
    out = torch.empty((tokens, h), dtype=torch.int16, device=dev)
    ga_mlp, ga_dn = 2688.0 / 0.6, 2688.0 / 0.05   # static input divisors (checkpoint-style constants)

    def run(st):
        for (wq, wqs), (wo, wos), (wf, wfs, gg, gu), (wd, wds, gd) in weights:
            lib.gemb_fp8_quantize(x, 1, xq, xs, tokens, h, st)
            lib.gemb_fp8_gemm_bf16(xq, xs, wq, wqs, y_qkv, tokens, qkv, h, st)
            lib.gemb_fp8_quantize(attn, 1, aq, as_, tokens, ao, st)
            lib.gemb_fp8_gemm_bf16(aq, as_, wo, wos, y_o, tokens, h, ao, st)
            lib.gemb_nvfp4_quantize(y_o, 1, oq, os_, tokens, h, ga_mlp, 1, 0, st)
            lib.gemb_nvfp4_gemm_gated_quant(oq, os_, wf, wfs, pq, ps, tokens, inter, h, ga_mlp, gg, gu, ga_dn, st)
            lib.gemb_nvfp4_gemm_bf16(pq, ps, wd, wds, out, tokens, h, inter, ga_dn, gd, st)

    (secs, clocks) = sampled(lambda: graph_time(run, 7 * layers, reps=5), dev.index or 0)
    lib.gemb_check_device_status()
    fp8_flops = 2.0 * tokens * (qkv * h + h * ao)
    fp4_flops = 2.0 * tokens * 3 * inter * h
    return {"metric": "prefill linear stack TFLOP/s", "workload": f"{layers} layers x 16,384 tokens: FP8 QKV+O, NVFP4 gate/up (fused GELU epilogue) + down, quantisers timed",
            "ms_per_stack": secs * 1e3, "ms_per_layer": secs * 1e3 / layers, "tokens_per_s": tokens / secs,
            "tflops_total": (fp8_flops + fp4_flops) * layers / secs / 1e12, "timed_region_s": secs * 5, "clocks": clocks,
            "flops_per_layer": {"fp8": fp8_flops, "nvfp4": fp4_flops},
            "ideal_ms_per_layer_at_nominal_peaks": (fp8_flops / 4.5e15 + fp4_flops / 9e15) * 1e3}


def bench_moe_layer(lib, dev, args=None, tokens=4096):
    """One 26B-A4B-like MoE layer on 4,096 tokens through gemb_moe_layer_forward (one CUDA graph)."""
    import torch
    from gem16_b200.moe import MoeLayer, synthetic_weights
    fused = True if args is None else args.fused
    w = synthetic_weights(dev, SEED + 3000)
    gen = torch.Generator(device=dev)
    gen.manual_seed(SEED + 3001)
    x = torch.randn((tokens, 2816), device=dev, generator=gen).to(torch.bfloat16)
    ga = float(2688.0 / x.float().abs().max().item())
    layer = MoeLayer(w, tokens, 8, ga, 2688.0 / 8.0, 2688.0 / 8.0, stages=False)
    layer.fused = fused
    xi = x.view(torch.int16)
    x_host = xi.cpu().pin_memory()
    out_host = torch.empty((tokens, 2816), dtype=torch.int16).pin_memory()
    st = torch.cuda.Stream(device=dev)
    graph = capture(st, lambda: layer.forward(xi, st))

    def region(fn, reps):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for _ in range(3):
            fn()
        st.synchronize()
        s.record(st)
        for _ in range(reps):
            fn()
        e.record(st)
        st.synchronize()
        return s.elapsed_time(e) / reps / 1e3

    def step_e2e():
        xi.copy_(x_host, non_blocking=True)
        graph.replay()
        out_host.copy_(layer.out, non_blocking=True)
        st.synchronize()

    with torch.cuda.stream(st):
        secs, clocks = sampled(lambda: region(graph.replay, 1200), dev.index or 0)
        secs_e2e = region(step_e2e, 100)
        stage_us = {}
        for sname, bit in STAGE_BITS.items():
            if (sname == "gelu" and fused) or sname == "exchange":
                continue
            lib.gemb_set_tuning(7, bit)
            try:
                g = capture(st, lambda: layer.forward(xi, st))
                stage_us[sname] = region(g.replay, 50) * 1e6
            finally:
                lib.gemb_set_tuning(7, 0)
    lib.gemb_check_device_status()
    fl = moe_layer_flops(tokens)
    flops = sum(fl.values())
    weight_bytes = moe_layer_weight_bytes()
    peaks = measured_peaks()
    gate_flops = tokens * 8 * 2.0 * 2 * 704 * 2816
    res = {"metric": "MoE layer tokens/s", "workload": f"moe_layer {tokens} tokens, 128 experts top-8, hidden 2816, expert 704, shared 2112",
           "value": tokens / secs, "unit": "tokens/s", "us_per_layer": secs * 1e6, "dtype": "nvfp4 (W4A4, fp32 accumulate)",
           "fused_gelu_epilogue": bool(fused), "timed_region_s": secs * 1200, "clocks": clocks,
           "e2e": {"value": tokens / secs_e2e, "unit": "tokens/s", "h2d_bytes_per_step": tokens * 2816 * 2, "d2h_bytes_per_step": tokens * 2816 * 2},
           "stage_us": stage_us, "flops": flops, "achieved_tflops": flops / secs / 1e12, "weight_bytes": weight_bytes,
           "bounds_us": {"tensor_at_9PF": flops / 9e15 * 1e6, "hbm_weights_at_measured_peak": weight_bytes / (peaks["hbm_gbs"] * 1e9) * 1e6},
           "roofline": {"bound": "tensor", "kernel": "gemm_kernel<nvfp4, grouped 128x256> gate/up" + (" + GELU requantising epilogue" if fused else ""),
                        "achieved": gate_flops / (stage_us["gate_up"] * 1e-6) / 1e12, "peak": FP4_NOMINAL_TFLOPS, "unit": "TFLOP/s",
                        "frac": gate_flops / (stage_us["gate_up"] * 1e-6) / 1e12 / FP4_NOMINAL_TFLOPS,
                        "peak_source": "nominal dense NVFP4 (9 PFLOP/s): no measured FP4 peak exists for this pool",
                        "avg_launch_us": stage_us["gate_up"], "time_x_sm_mhz": stage_us["gate_up"] * (clocks["sm_mhz"] or 0)},
           "padded_rows": int(layer.plan[1].item()), "tiles": int(layer.plan[0].item()),
           "expert_count_max": int(layer.counts.max().item()), "expert_count_min": int(layer.counts.min().item())}
    if args is None or not args.no_cpu_baseline:
        dt, cores, kind = cpu_moe_layer_sample(use_ref=True, tokens=64)
        res["cpu_baseline"] = {"value": 64 / dt, "unit": "tokens/s", "cores": cores, "kind": kind,
                               "sample": f"64 of the {tokens} tokens through the layer: {dt:.2f} s on {cores} host threads"}
    return res


def bench_output_head(lib, dev, args=None, vocab=262144, hidden=3840):
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


def bench_verifier_gemv(lib, dev, args=None, sets=6):
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


def sampled(fn, index=0):
    """fn() with the SM clock sampled beside it: (result, clocks)."""
    s = ClockSampler(index).start()
    r = fn()
    return r, s.stop()


def bench_decode_gemv(lib, dev, args):
    """The decode GEMV set: 48 layers x four FP8 projections (gate/up, down, QKV, O), bf16 activations
    quantised per token, 48 distinct weight sets (10.8 GB >> L2), one CUDA graph per pass."""
    import torch
    layers = args.layers
    gen = torch.Generator(device=dev)
    gen.manual_seed(SEED + 1000)
    weights = []
    for _ in range(layers):
        mats = []
        for _, rows, k in DECODE_SHAPES:
            w = torch.randn((rows, k), device=dev, dtype=torch.float32, generator=gen) * 0.02
            wq = torch.empty((rows, k), device=dev, dtype=torch.uint8)
            wsc = torch.empty((rows,), device=dev, dtype=torch.float32)
            lib.gemb_fp8_quantize(w, 0, wq, wsc, rows, k, None)
            mats.append((wq, wsc.to(torch.bfloat16).view(torch.int16)))
            del w
        weights.append(mats)
    x_elems = sum(k for _, _, k in DECODE_SHAPES) * layers
    y_elems = sum(r for _, r, _ in DECODE_SHAPES) * layers
    x_host = torch.randn((x_elems,), dtype=torch.float32).to(torch.bfloat16).pin_memory()
    x_dev = x_host.to(dev)
    xq_dev = torch.empty((x_elems,), dtype=torch.uint8, device=dev)
    xs_dev = torch.empty((layers * len(DECODE_SHAPES),), device=dev)
    y_dev = torch.zeros((y_elems,), device=dev)
    y_host = torch.empty((y_elems,), dtype=torch.float32).pin_memory()

    def enqueue(st, quantize=True):
        xo = yo = n = 0
        for mats in weights:
            for (wq, ws), (_, rows, k) in zip(mats, DECODE_SHAPES):
                if quantize:
                    lib.gemb_fp8_quantize(x_dev[xo:xo + k], 1, xq_dev[xo:xo + k], xs_dev[n:n + 1], 1, k, st)
                lib.gemb_fp8_gemv(xq_dev[xo:xo + k], xs_dev[n:n + 1], wq, ws, y_dev[yo:yo + rows], rows, k, st)
                xo += k
                yo += rows
                n += 1
        return n

    def enqueue_fused(st):
        """One launch per projection: the token quantizer inside the GEMV (bit-identical to the pair)."""
        xo = yo = 0
        for mats in weights:
            for (wq, ws), (_, rows, k) in zip(mats, DECODE_SHAPES):
                lib.gemb_fp8_gemv_bf16in(x_dev[xo:xo + k], wq, ws, y_dev[yo:yo + rows], 0, rows, k, st)
                xo += k
                yo += rows

    st = torch.cuda.Stream(device=dev)
    launches = 2 * layers * len(DECODE_SHAPES)
    full = capture(st, lambda: enqueue(st))
    only = capture(st, lambda: enqueue(st, quantize=False))
    fused = capture(st, lambda: enqueue_fused(st))

    def region(g, reps):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for _ in range(3):
            g()
        st.synchronize()
        s.record(st)
        for _ in range(reps):
            g()
        e.record(st)
        st.synchronize()
        return s.elapsed_time(e) / reps / 1e3

    def step_e2e():
        x_dev.copy_(x_host, non_blocking=True)
        full.replay()
        y_host.copy_(y_dev, non_blocking=True)
        st.synchronize()

    with torch.cuda.stream(st):
        reps = max(20, int(0.6 / 2.6e-3))
        secs, clocks = sampled(lambda: region(full.replay, reps), dev.index or 0)
        secs_gemv = region(only.replay, reps)
        secs_fused = region(fused.replay, reps)
        secs_e2e = region(step_e2e, 20)
    lib.gemb_check_device_status()
    bytes_pass = decode_bytes_per_layer() * layers
    peaks = measured_peaks()
    per_launch = bytes_pass / (launches // 2)
    achieved = bytes_pass / secs_gemv / 1e9
    prof = profile_traffic("fp8_gemv_kernel_decode.md")
    out = {"metric": "decode GEMV GB/s", "workload": "decode_gemv: 48 layers x (gate/up 3840->30720, down 15360->3840, QKV 3840->8192, O 4096->3840), FP8 W8A8",
           "value": bytes_pass / secs / 1e9, "unit": "GB/s", "ms_per_pass": secs * 1e3, "dtype": "fp8_e4m3 (fp32 accumulate)",
           "timed_region_s": secs * reps, "clocks": clocks, "launches_per_pass": launches,
           "e2e": {"value": bytes_pass / secs_e2e / 1e9, "unit": "GB/s", "h2d_bytes_per_step": x_elems * 2, "d2h_bytes_per_step": y_elems * 4},
           "roofline": {"bound": "hbm", "kernel": "fp8_gemv_kernel", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                        "frac": achieved / peaks["hbm_gbs"], "peak_source": peaks["source"], "frac_of_nominal_8TBs": achieved / 8000.0,
                        "avg_launch_us": secs_gemv / (launches // 2) * 1e6, "algorithmic_bytes_per_launch": per_launch,
                        "traffic": (prof["traffic_bytes_per_launch"] * per_launch / prof["captured_units_per_launch"])
                        if prof and prof.get("captured_units_per_launch") else None,
                        "traffic_unit": "dram bytes per launch, scaled from the kept ncu capture by algorithmic bytes",
                        "whole_pass": {"kernels": "fp8_quantize_decode_kernel + fp8_gemv_kernel", "achieved": bytes_pass / secs / 1e9,
                                       "frac": bytes_pass / secs / 1e9 / peaks["hbm_gbs"]},
                        "whole_pass_quantizer_in_gemv": {"kernels": "gemb_fp8_gemv_bf16in: one launch per projection, same bits",
                                                         "ms_per_pass": secs_fused * 1e3, "achieved": bytes_pass / secs_fused / 1e9,
                                                         "frac": bytes_pass / secs_fused / 1e9 / peaks["hbm_gbs"]}},
           "l2": f"{layers} distinct weight sets, {bytes_pass / 1e9:.2f} GB per pass >> 126 MB L2", "multi_gpu": "replicas only"}
    if not args.no_cpu_baseline:
        gbs, dt, cores, kind = cpu_decode_sample(1, 0, use_ref=True)
        out["cpu_baseline"] = {"value": gbs, "unit": "GB/s", "cores": cores, "kind": kind,
                               "sample": f"one decode layer of 48 (224 MB), {dt:.2f} s on {cores} host threads"}
    del weights, full, only, fused
    torch.cuda.empty_cache()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-other-workloads", action="store_true")
    ap.add_argument("--no-stage-times", action="store_true")
    ap.add_argument("--unfused", dest="fused", action="store_false",
                    help="gate/up GEMM, GELU requantisation as separate launches instead of the fused epilogue")
    ap.add_argument("--ep-shared-sms", type=int, default=None,
                    help="N > 1: SMs the shared branch gets beside the pushing down GEMM (GEMB_TUNE_EP_SHARED_SMS; default: the library's)")
    ap.add_argument("--ep-split-sms", type=int, default=None,
                    help="N > 1: two-half schedule with the first half's push on this many SMs (GEMB_TUNE_EP_SPLIT_SMS)")
    ap.add_argument("--moe-layers", type=int, default=MOE_LAYERS,
                    help="MoE layers held on the device (30 = the benchmark; fewer for a small profiler capture)")
    ap.add_argument("--layers", type=int, default=LAYERS,
                    help="decode layers held on the device (48 = the benchmark; fewer for a small profiler capture)")
    ap.add_argument("--only", default=None, choices=["decode_gemv", "nvfp4_linear", "moe_layer", "prefill_gemm", "prefill_stack",
                                                     "output_head", "verifier_gemv"],
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
        fn = {"decode_gemv": bench_decode_gemv, "nvfp4_linear": bench_nvfp4_linear, "moe_layer": bench_moe_layer,
              "prefill_gemm": bench_prefill_gemm, "prefill_stack": bench_prefill_stack, "output_head": bench_output_head,
              "verifier_gemv": bench_verifier_gemv}[args.only]
        emit(fn(load(), dev, args))
        return
    moe_headline(args)


if __name__ == "__main__":
    main()
