#!/usr/bin/env python
"""Benchmark of the xnor conv path on B200.  Default workload: yolov3-tiny_xnor forward at 416x416, batch 1 per GPU.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
                    [--workload NET] [--batch B | --global-batch B] [--forwards-per-step F]
    python bench.py --kernel gemm --shape M N K [--route auto|integer|tensor|tiled] [--tc-kernel 1|2] [--shortcut] [--reps R] [--no-graph]
    python bench.py --kernel layer --shape BATCH C H W N KS [STRIDE] [--sum-only] [--route ...] [--tc-kernel 1|2]
    python bench.py --kernel pack --shape BATCH C H W N KS [--pack-ctas-per-sm C] [--reps R] [--no-graph]
    python bench.py --kernel gemms | --kernel fconv --shape CASE

One forward is one pass of the network over one batch of seeded synthetic input with seeded random weights (no
dataset or checkpoint is involved), captured once into a CUDA graph and replayed.  One STEP is `forwards_per_step`
forwards (stated in `config`), so that a 20-step run times well over 100 ms; every forward is timed with its own
pair of CUDA events on the launch stream and the L2 is flushed between forwards, outside the intervals.

Printed JSON (one line, rank 0):
  value         images/s, inputs resident in HBM (sum of the per-forward event intervals, max over ranks)
  e2e           images/s with the input copied from pinned host memory and the head outputs copied back inside the
                timed region; e2e.blocking_call = the same through a blocking predict call (copy in, forward, copy
                out, stream synchronise per call) timed with the host clock, e2e.double_buffered = that loop
                with the next input's copy overlapping the current forward, and e2e.streamed = the same with the
                host synchronising only after the last call
  roofline*     single kernels timed alone against a peak measured in the same run (integer XOR+POPC+ADD issue
                rate, tcgen05 kind::mxf4 and kind::i8 rates) or MEASURED_PEAKS.json (HBM): the calls rotate over
                copies of their buffers that together exceed twice the L2, and a whole rotation is one CUDA graph
                between two events
  gpu_reference the reference's own GPU xnor kernels compiled for sm_100a (oracle/_ref) beside this library's
                layer call on BASELINE configuration 1
  cpu_baseline  the reference's own CPU xnor code (oracle/_ref) on the same layer shapes, all host cores and one

--impl reference times only that CPU code (xnor layers of the same network) and prints its own line.
With N > 1 (torchrun) every rank runs an independent replica on its GPU: replicas only, no collective on the data
path; NCCL is used for the barrier and the max over ranks.  --global-batch cuts one batch over the ranks instead.
--kernel runs one kernel of the library on random operands and prints its median time, measured like the roofline
legs; with --no-graph the calls are launched directly (the form the profiler captures are made with).
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

METRIC = "images/s yolov3-tiny_xnor@416"
L2_FLUSH_BYTES = 256 << 20
L2_BYTES = 126 << 20
TARGET_STEP_MS = 8.0
ROUTES = {"auto": 0, "integer": 1, "tensor": 2, "tiled": 3}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=40)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--batch", type=int, default=1, help="images per GPU per forward (the metric is quoted at 1)")
    ap.add_argument("--global-batch", type=int, default=0,
                    help="images per forward over ALL GPUs, cut into per-rank slices (strong scaling; BASELINE configurations 4 "
                         "and 5); 0 = --batch images on every GPU (weak scaling, the default)")
    ap.add_argument("--forwards-per-step", type=int, default=0,
                    help="forward passes that make up one step (0 = as many as bring a step to about 8 ms, at least 1)")
    ap.add_argument("--cpu-baseline-seconds", type=float, default=12.0)
    ap.add_argument("--workload", default="yolov3-tiny_xnor", choices=["yolov3-tiny_xnor", "tiny-yolo_xnor", "darknet53_448_xnor"],
                    help="network to run; the default is the configuration the metric is quoted on, the others are the "
                         "batched BASELINE configurations (use with --batch or --global-batch)")
    ap.add_argument("--kernel", default=None, choices=["gemm", "gemms", "pack", "fconv", "layer"], help="time one kernel instead of the network")
    ap.add_argument("--sum-only", action="store_true", help="--kernel layer: only the sum with a fused shortcut operand is written, plus its sign words")
    ap.add_argument("--shape", type=int, nargs="*", default=[])
    ap.add_argument("--route", default="auto", choices=sorted(ROUTES))
    ap.add_argument("--tc-kernel", type=int, default=0, choices=[0, 1, 2], help="--kernel gemm with --route tensor: 1 = one tile per CTA, 2 = persistent")
    ap.add_argument("--shortcut", action="store_true")
    ap.add_argument("--reps", type=int, default=5)
    ap.add_argument("--pack-ctas-per-sm", type=int, default=0, help="--kernel pack: CTAs per SM the pack kernels size their grid for (0 = default)")
    ap.add_argument("--no-graph", action="store_true", help="--kernel: launch directly instead of replaying a captured graph (for profiler captures)")
    return ap.parse_args()


def workload_text(name: str, size: int, batch_text: str) -> str:
    return f"{name} forward, {size}x{size}x3 fp32 input U[0,1), {batch_text}, seeded random weights"


# ---- CPU reference arm ---------------------------------------------------------------------------

def xnor_layer_table(workload: str):
    import torch  # noqa: F401  (network.py imports torch; CPU only here)
    from darknet_b200 import cfgs, network
    with tempfile.TemporaryDirectory() as td:
        p = os.path.join(td, "net.cfg")
        with open(p, "w") as fh:
            fh.write(cfgs.CFGS[workload]())
        net = network.parse_network_cfg(p, 1, "cpu")
    # bin_output layers lose their activation at load (calculate_binary_weights)
    rows = network.xnor_layer_shapes(net)
    for r, l in zip(rows, [l for l in net.layers if l.type == "convolutional" and l.xnor]):
        r["leaky"] = int(l.activation == "leaky" and not l.use_bin_output)
    return rows, net.h


class CpuReference:
    """The reference's CPU xnor forward (oracle/_ref: its own sources compiled unmodified, preferably the build with the
    reference's own optimisation flags) over the xnor layers of the workload; where neither build is present, the plain-C
    restatement.  Built once, then timed."""

    def __init__(self, workload: str, threads: int | None = None) -> None:
        import synth
        from oracle import binding
        self.workload = workload
        self.rows, self.size = xnor_layer_table(workload)
        self.cores = threads or os.cpu_count() or 1
        fast = getattr(binding, "REF_FAST_SO", None)
        if fast and os.path.exists(fast):
            self.ref, self.kind = binding.Ref(fast), "reference"
            self.build = "reference flags (-O3 -ffp-contract=fast -funsafe-math-optimizations, AVX2)"
        elif binding.Ref.available():
            self.ref, self.kind, self.build = binding.Ref(), "reference", "checker flags (-O3, AVX2, no fast-math)"
        else:
            self.ref, self.kind, self.build = None, "port", "plain-C restatement"
        if self.ref is not None:
            self.ref.set_gpu_index(-1)
            self.ref.set_num_threads(self.cores)
            self.layers = []
            for i, r in enumerate(self.rows):
                x, wt, b = synth.conv_case(900 + i, 1, r["c"], r["h"], r["w"], r["n"], r["size"])
                self.layers.append((self.ref.layer((r["c"], r["h"], r["w"]), wt, b, r["stride"], r["pad"], bool(r["leaky"])), x[0]))
            self._one = lambda: [lay.forward(x) for lay, x in self.layers]
        else:
            port = binding.Port()
            cases = [(synth.conv_case(900 + i, 1, r["c"], r["h"], r["w"], r["n"], r["size"]), r) for i, r in enumerate(self.rows)]
            self._one = lambda: [port.conv_forward(x, wt, b, r["stride"], r["pad"], r["leaky"]) for (x, wt, b), r in cases]
        self._one()  # warm-up (page-in, OpenMP pool)

    def set_threads(self, n: int) -> None:
        self.cores = n
        if self.ref is not None:
            self.ref.set_num_threads(n)
        self._one()

    def run(self, images: int) -> float:
        """Seconds for `images` single-image forwards of all xnor layers."""
        t0 = time.perf_counter()
        for _ in range(images):
            self._one()
        return time.perf_counter() - t0

    def images_for(self, seconds: float) -> int:
        t = max(self.run(1), 1e-6)
        return max(1, int(seconds / t))

    def describe(self, images: int, seconds: float) -> str:
        return (f"{images} images x {len(self.rows)} xnor layers of {self.workload}@{self.size} (float layers excluded), "
                f"{seconds:.1f} s, {self.cores} threads, {self.build}")


def time_cpu_reference(workload: str, budget_s: float):
    cpu = CpuReference(workload)
    n = cpu.images_for(budget_s * 0.7)
    el = cpu.run(n)
    all_cores = {"value": n / el, "unit": "images/s", "cores": cpu.cores, "kind": cpu.kind, "sample": cpu.describe(n, el)}
    if cpu.ref is not None:
        cpu.set_threads(1)
        n1 = cpu.images_for(budget_s * 0.3)
        el1 = cpu.run(n1)
        all_cores["one_thread"] = {"value": n1 / el1, "unit": "images/s", "cores": 1, "sample": cpu.describe(n1, el1)}
    return all_cores


def run_reference_arm(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cpu = CpuReference(args.workload)
    per_step = max(0.2, min(2.0, 150.0 / max(args.steps + args.warmup, 1)))
    n = cpu.images_for(per_step)        # images per step: a bounded sample of the workload
    for _ in range(args.warmup):
        cpu.run(n)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu.run(n)
    el = time.perf_counter() - t0
    value = n * args.steps / el
    default = (args.workload == "yolov3-tiny_xnor")
    if args.global_batch:
        batch_text = f"global batch {args.global_batch} cut over {args.gpus} GPU(s)"
    else:
        batch_text = f"batch {args.batch} per GPU"
    line = {
        "impl": "reference", "metric": METRIC if default else f"images/s {args.workload}@{cpu.size}", "value": value, "unit": "images/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1000.0 * el / args.steps,
        "higher_is_better": True, "scaling": "strong" if args.global_batch else "weak", "vs_baseline": None, "dtype": "u32",
        "data": "synthetic",
        "config": {"workload": workload_text(args.workload, cpu.size, batch_text)},
        "reference_scope": {"layers": "xnor conv layers only (the path), reference CPU code on host cores, one image at a time as the reference runs it",
                            "images_per_step": n},
        "cpu_baseline": {"value": value, "unit": "images/s", "cores": cpu.cores, "kind": cpu.kind,
                         "sample": cpu.describe(n * args.steps, el)},
        "e2e": {"value": value, "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ---- GPU arm -------------------------------------------------------------------------------------

class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int) -> None:
        self.proc = None
        self.path = tempfile.NamedTemporaryFile(prefix="clocks_", suffix=".csv", delete=False).name
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={gpu_index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for row in open(self.path).read().splitlines():
            f = [v.strip() for v in row.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.path)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def captured_traffic(key: str):
    """DRAM bytes (read + write) of one launch as an ncu capture recorded them.  profiles/dram_traffic.json, written when
    a capture is summarised, holds per entry the kernel, its shape, the bytes and the date.  (None, None) when absent."""
    try:
        table = json.load(open(os.path.join(ROOT, "profiles", "dram_traffic.json")))
        e = table[key]
        return float(e["bytes_per_launch"]), f"ncu capture of {e['kernel']} ({e['shape']}), {e['captured']}"
    except (OSError, ValueError, KeyError):
        return None, None


def device_status(capi) -> int:
    st = C.c_int(-1)
    capi.check(capi.lib().xnor_b200_take_device_status(C.byref(st)), "xnor_b200_take_device_status")
    return st.value


def run_gpu_arm(args) -> None:
    import torch
    import torch.distributed as dist
    import synth
    from darknet_b200 import capi, cfgs, network, replicas

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback for the xnor path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    capi.lib()  # fail loudly if the CUDA library is missing

    if args.global_batch:
        first_image, batch = replicas.shard_batch(args.global_batch, world)[rank]
        if batch == 0:
            raise SystemExit("bench: --global-batch must give every rank at least one image")
        images_per_forward = args.global_batch
    else:
        first_image, batch = rank * args.batch, args.batch
        images_per_forward = world * batch
    with tempfile.TemporaryDirectory() as td:
        cfg_path, w_path = os.path.join(td, "net.cfg"), os.path.join(td, "synthetic.weights")
        with open(cfg_path, "w") as fh:
            fh.write(cfgs.CFGS[args.workload]())
        net0 = network.parse_network_cfg(cfg_path, batch, "cpu")
        network.write_synthetic_weights(net0, w_path, seed=1)
        net = network.load_network_custom(cfg_path, w_path, batch, str(dev))
    rows = network.xnor_layer_shapes(net)
    binops_per_image = sum(r["binops"] for r in rows)

    default_workload = (args.workload == "yolov3-tiny_xnor")
    batch_text = f"global batch {args.global_batch} cut over {world} GPU(s)" if args.global_batch else f"batch {batch} per GPU"
    metric_text = METRIC if default_workload else f"images/s {args.workload}@{net.h}"
    # image i of the global batch is the same tensor whatever the number of ranks
    x_host = torch.from_numpy(np.concatenate([synth.uniform01(1 + first_image + i, (1, 3, net.h, net.w)) for i in range(batch)], 0)).pin_memory()
    x_dev = x_host.to(dev, non_blocking=True)
    stream = torch.cuda.Stream(dev)
    flush = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device=dev)

    # warm-up outside capture (cuDNN autotune, shared-memory attributes), then capture one forward
    with torch.cuda.stream(stream):
        for _ in range(3):
            heads = network.forward_network_gpu(net, x_dev)
    stream.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        heads = network.forward_network_gpu(net, x_dev)
    head_host = [torch.empty(h.shape, dtype=h.dtype).pin_memory() for h in heads]
    # the end-to-end forward as one graph: input copy from pinned memory, forward, every head copied to pinned memory on
    # the stream that produced it
    graph_e2e = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph_e2e, stream=stream):
        x_dev.copy_(x_host, non_blocking=True)
        network.forward_network_gpu(net, x_dev, head_host)
    h2d_bytes = x_host.numel() * 4
    d2h_bytes = sum(h.numel() * 4 for h in heads)

    def barrier():
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def timed_forwards(n: int, end_to_end: bool) -> float:
        """Total milliseconds of n forwards (sum of per-forward CUDA-event intervals; the L2 flush between forwards sits
        outside the intervals)."""
        total = 0.0
        while n > 0:
            chunk = min(n, 512)
            evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(chunk)]
            with torch.cuda.stream(stream):
                for a, b in evs:
                    flush.fill_(1)
                    a.record(stream)
                    (graph_e2e if end_to_end else graph).replay()
                    b.record(stream)
            stream.synchronize()
            total += float(sum(a.elapsed_time(b) for a, b in evs))
            n -= chunk
        return total

    fps = args.forwards_per_step
    if fps <= 0:
        probe_ms = replicas.max_over_ranks(timed_forwards(5, False) / 5.0, dev)
        fps = max(1, int(round(TARGET_STEP_MS / max(probe_ms, 1e-3))))
    sampler = ClockSampler(local) if rank == 0 else None
    timed_forwards(args.warmup * fps, False)
    barrier()
    ms_total = timed_forwards(args.steps * fps, False)
    barrier()
    ms_total = replicas.max_over_ranks(ms_total, dev)
    timed_forwards(max(3, args.warmup) * fps, True)
    barrier()
    ms_e2e = timed_forwards(args.steps * fps, True)
    barrier()
    ms_e2e = replicas.max_over_ranks(ms_e2e, dev)
    for hh, hd in zip(head_host, heads):               # what the end-to-end forwards left in pinned host memory = the device-resident forward
        if not torch.equal(hh, hd.cpu()):
            raise SystemExit("bench: host copy of a head differs from the device tensor")
    clocks = sampler.stop() if sampler else None

    # The same end-to-end forward as a blocking predict call (Darknet's network_predict_gpu pushes the input, runs the
    # layers and synchronises the stream once per call, src-lib/network_kernels.cu:748-761), timed with the host clock.
    n_block = max(20, min(args.steps * fps, 400))

    def blocking_calls(n: int) -> float:
        with torch.cuda.stream(stream):
            t0 = time.perf_counter()
            for _ in range(n):
                graph_e2e.replay()
                stream.synchronize()
            return time.perf_counter() - t0

    blocking_calls(5)
    barrier()
    wall_block = replicas.max_over_ranks(blocking_calls(n_block), dev)
    # Double-buffered variant: a second input buffer and copy stream; the copy of input i+1 runs under forward i.  The
    # forward graph reads x_dev, so the staged input is moved into it device-to-device at the start of each forward.
    copy_stream = torch.cuda.Stream(dev)
    x_stage = torch.empty_like(x_dev)

    def double_buffered(n: int, sync_every_call: bool = True) -> float:
        staged, consumed = torch.cuda.Event(), torch.cuda.Event()
        with torch.cuda.stream(copy_stream):
            x_stage.copy_(x_host, non_blocking=True)
            staged.record(copy_stream)
        t0 = time.perf_counter()
        for i in range(n):
            with torch.cuda.stream(stream):
                stream.wait_event(staged)
                x_dev.copy_(x_stage, non_blocking=True)
                consumed.record(stream)
                graph.replay()
                for hh, hd in zip(head_host, heads):
                    hh.copy_(hd, non_blocking=True)
            if i + 1 < n:
                with torch.cuda.stream(copy_stream):
                    copy_stream.wait_event(consumed)
                    x_stage.copy_(x_host, non_blocking=True)
                    staged.record(copy_stream)
            if sync_every_call:
                stream.synchronize()
        stream.synchronize()
        return time.perf_counter() - t0

    double_buffered(5)
    barrier()
    wall_db = replicas.max_over_ranks(double_buffered(n_block), dev)
    double_buffered(5, False)
    barrier()
    wall_stream = replicas.max_over_ranks(double_buffered(n_block, False), dev)
    status = device_status(capi)
    if status != 0:
        raise SystemExit(f"bench: the tensor-core GEMM reported device status {status} (a bounded wait ran out); the timings are void")

    value = images_per_forward * args.steps * fps / (ms_total * 1e-3)
    e2e_value = images_per_forward * args.steps * fps / (ms_e2e * 1e-3)

    # ---- rooflines of single kernels, rank 0 only ----
    extra = {}
    cpu_baseline = None
    roofline = None
    if rank == 0 and default_workload and not args.global_batch:
        extra, roofline = kernel_rooflines(net, batch, binops_per_image, stream, flush, dev)
        if world == 1:
            cpu_baseline = time_cpu_reference(args.workload, args.cpu_baseline_seconds)

    if rank == 0:
        line = {
            "metric": metric_text, "value": value, "unit": "images/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_total / args.steps, "higher_is_better": True, "scaling": "strong" if args.global_batch else "weak",
            "vs_baseline": None, "dtype": "u32", "data": "synthetic",
            "config": {"workload": workload_text(args.workload, net.h, batch_text), "global_batch": images_per_forward,
                       "forwards_per_step": fps, "images_per_step": images_per_forward * fps,
                       "folded_maxpools": net.folded_maxpools, "sign_sinks": net.sink_links, "sign_links": net.sign_links,
                       "side_branch": any(l.branch_start for l in net.layers), "parallelism": f"replicas x{world} (no collective)",
                       "l2": "256 MiB buffer written between timed forwards", "timing": "per-forward CUDA events on the launch stream, CUDA graph replay",
                       "float_layers": "this library's fp32 kernels at small batch (first conv + pool + sign, small-map convs with the yolo activation), cuDNN/ATen otherwise",
                       "xnor_binops_per_image": binops_per_image},
            "xnor_gemm_tops": roofline["achieved"] if roofline else None,
            "roofline": roofline, **extra,
            "cpu_baseline": cpu_baseline,
            "e2e": {"value": e2e_value, "unit": "images/s", "h2d_bytes_per_step": h2d_bytes * fps, "d2h_bytes_per_step": d2h_bytes * fps,
                    "ms_per_step": ms_e2e / args.steps,
                    "blocking_call": {"value": images_per_forward * n_block / wall_block, "unit": "images/s", "ms_per_call": 1000.0 * wall_block / n_block,
                                      "timing": "host clock around copy-in + forward + copy-out + stream synchronise per call", "calls": n_block},
                    "double_buffered": {"value": images_per_forward * n_block / wall_db, "unit": "images/s", "ms_per_call": 1000.0 * wall_db / n_block,
                                        "timing": "host clock; the next input's host-to-device copy overlaps the current forward", "calls": n_block},
                    "streamed": {"value": images_per_forward * n_block / wall_stream, "unit": "images/s", "ms_per_call": 1000.0 * wall_stream / n_block,
                                 "timing": "host clock over the whole run; as double_buffered, but the host only synchronises after the last call "
                                           "(a stream of images whose results are read later)", "calls": n_block}},
            "gpu_launches": args.steps * fps * network.own_launches_per_forward(net),
            "device_status": status,
            "max_memory_gb": torch.cuda.max_memory_allocated(dev) / 1e9,
            "clocks": clocks,
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def kernel_rooflines(net, batch, binops_per_image, stream, flush, dev):
    """Single kernels timed alone, against measured peaks: the calls rotate over copies of their buffers that together exceed
    twice the L2 and a whole rotation is one CUDA graph between two events (see time_rotating)."""
    import torch
    import synth
    from darknet_b200 import capi
    from darknet_b200 import layer as L
    lib = capi.lib()
    xl_layers = [l.xnor_layer for l in net.layers if l.type == "convolutional" and l.xnor]
    inputs = [torch.from_numpy(synth.bell(50 + i, (batch, xl.c, xl.h, xl.w))).to(dev) for i, xl in enumerate(xl_layers)]
    packed = [L.pack_input(xl, xi) for xl, xi in zip(xl_layers, inputs)]
    torch.cuda.synchronize(dev)
    reps = 50

    def time_rotating(calls) -> float:
        """Average ms of ONE of `calls`.  They do the same work on separate copies of their buffers whose total size is
        more than twice the L2, so every call finds its operands in HBM; all of them are captured, in order, into one
        CUDA graph, and a sweep of the graph is timed between two events -- neither host launch overhead nor the few
        microseconds an event pair costs by itself end up in a single call's figure."""
        with torch.cuda.stream(stream):
            for fn in calls:
                fn()
        stream.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            for fn in calls:
                fn()
        evs = []
        with torch.cuda.stream(stream):
            for _ in range(3):
                g.replay()
            for _ in range(reps):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(stream)
                g.replay()
                b.record(stream)
                evs.append((a, b))
        stream.synchronize()
        return sum(a.elapsed_time(b) for a, b in evs) / reps / len(calls)

    def copies_for(set_bytes: int) -> int:
        return max(2, -(-int(2.2 * L2_BYTES) // max(int(set_bytes), 1)))

    def cur() -> int:
        return torch.cuda.current_stream().cuda_stream

    set_bytes = sum(xl.align_bit_weights_gpu.numel() + pk.numel() + 4 * xl.n * batch * xl.geom.n_out for xl, pk in zip(xl_layers, packed))
    n_sets = copies_for(set_bytes)
    weight_sets = [[xl.align_bit_weights_gpu.clone() for xl in xl_layers] for _ in range(n_sets)]
    packed_sets = [[pk.clone() for pk in packed] for _ in range(n_sets)]
    output_sets = [[torch.empty(xl.n, batch * xl.geom.n_out, device=dev) for xl in xl_layers] for _ in range(n_sets)]
    n_in_sets = copies_for(sum(4 * xi.numel() + pk.numel() for xi, pk in zip(inputs, packed)))
    input_sets = [[xi.clone() for xi in inputs] for _ in range(n_in_sets)]

    def all_gemms(i):
        def run():
            for xl, w, pk, o in zip(xl_layers, weight_sets[i], packed_sets[i], output_sets[i]):
                g = xl.geom
                capi.check(lib.xnor_b200_gemm_bin_mean_transposed(
                    xl.n, batch * g.n_out, g.k, w.data_ptr(), g.new_lda, pk.data_ptr(), g.new_lda,
                    o.data_ptr(), batch * g.n_out, xl.mean_arr_gpu.data_ptr(), xl.biases_gpu.data_ptr(),
                    int(xl.activation == capi.LEAKY), None, None, cur()), "gemm")
        return run

    def all_packs(i):
        def run():
            for xl, xi, pk in zip(xl_layers, input_sets[i], packed_sets[i % n_sets]):
                capi.check(lib.xnor_b200_pack_input(C.byref(xl.desc), xi.data_ptr(), pk.data_ptr(), cur()), "pack")
        return run

    ms_gemm = time_rotating([all_gemms(i) for i in range(n_sets)])
    ms_pack = time_rotating([all_packs(i) for i in range(n_in_sets)])
    del weight_sets, output_sets, input_sets
    g_, m_ = C.c_double(), C.c_double()
    capi.check(lib.xnor_b200_measure_popc_peak(20000, C.byref(g_), C.byref(m_)), "popc peak")
    popc_peak_tops = g_.value / 1e3
    capi.check(lib.xnor_b200_measure_bmma_peak(2000, C.byref(g_), C.byref(m_)), "bmma peak")
    bmma_peak_tops = g_.value / 1e3
    capi.check(lib.xnor_b200_measure_umma_i8_peak(4000, C.byref(g_), C.byref(m_)), "umma peak")
    umma_i8_peak_tops = g_.value / 1e3
    capi.check(lib.xnor_b200_measure_umma_mxf4_peak(4000, C.byref(g_), C.byref(m_)), "umma mxf4 peak")
    umma_peak_tops = g_.value / 1e3
    achieved = binops_per_image * batch / (ms_gemm * 1e-3) / 1e12
    traffic, traffic_source = captured_traffic("xnor_gemm_b1_yolov3_tiny_set") if batch == 1 else (None, None)
    roofline = {
        "kernel": "xnor GEMM kernels of one forward (9 launches = the xnor layers of yolov3-tiny_xnor, stand-alone calls with fp32 epilogue)",
        "bound": "int_popc", "achieved": achieved, "peak": popc_peak_tops, "unit": "TOP/s (binary ops, 2*M*N*K)",
        "frac": achieved / popc_peak_tops, "traffic": traffic, "traffic_source": traffic_source,
        "algorithmic_bytes": sum((xl.n + batch * xl.geom.n_out) * xl.geom.new_lda // 8 + 4 * xl.n * batch * xl.geom.n_out for xl in xl_layers),
        "peak_source": "measured in this run: register-resident XOR+POPC+ADD loop on all SMs",
        "b1_mma_sync_peak": bmma_peak_tops, "ms_per_forward": ms_gemm,
    }
    pack_bytes = sum(batch * (4 * xl.c * xl.h * xl.w + xl.geom.n_out * xl.geom.new_lda // 8) for xl in xl_layers)
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except (OSError, ValueError):
        pass
    hbm_peak = float(peaks.get("hbm_gbs", 6650.0))
    hbm_source = "MEASURED_PEAKS.json (of measured)" if peaks else "fallback 6650 GB/s (of fallback)"
    pack_gbs = pack_bytes / (ms_pack * 1e-3) / 1e9
    out = {"roofline_pack": {
        "kernel": "pack_input_*_kernel (9 launches: every xnor layer's stand-alone xnor_b200_pack_input; the linked forward replaces most of them by sign sinks)",
        "bound": "hbm", "achieved": pack_gbs, "peak": hbm_peak, "unit": "GB/s", "frac": pack_gbs / hbm_peak, "traffic": None,
        "ms_per_forward": ms_pack, "peak_source": hbm_source}}

    # BASELINE configuration 1 (256 -> 512 filters, 26x26, 3x3) at batch 64, one GEMM call, each route pinned in turn
    # through xnor_b200_set_tuning: the tcgen05 kernel against the kind::i8 rate, the integer kernels against the popc rate.
    M_, N_, K_ = 512, 64 * 676, 2304
    lda_ = K_ + (256 - K_ % 256)
    alg_big = (M_ + N_) * lda_ // 8 + 4 * M_ * N_
    n_big = copies_for(alg_big)
    A_ = torch.randint(0, 256, (M_, lda_ // 8), dtype=torch.uint8, device=dev)
    B_ = torch.randint(0, 256, (N_, lda_ // 8), dtype=torch.uint8, device=dev)
    A_[:, K_ // 8:] = 0
    B_[:, K_ // 8:] = 0
    As_ = [A_.clone() for _ in range(n_big)]
    Bs_ = [B_.clone() for _ in range(n_big)]
    Cs_ = [torch.empty(M_, N_, device=dev) for _ in range(n_big)]
    C_ = Cs_[0]
    mean_ = torch.rand(M_, device=dev)
    bias_ = torch.rand(M_, device=dev)

    def big_gemm(i):
        def run():
            capi.check(lib.xnor_b200_gemm_bin_mean_transposed(M_, N_, K_, As_[i].data_ptr(), lda_, Bs_[i].data_ptr(), lda_, Cs_[i].data_ptr(), N_,
                                                              mean_.data_ptr(), bias_.data_ptr(), 1, None, None, cur()), "gemm")
        return run
    big_gemms = [big_gemm(i) for i in range(n_big)]
    ops_big = 2.0 * M_ * N_ * K_
    capi.set_tuning(gemm_route=capi.ROUTE_TENSOR)
    ms_big = time_rotating(big_gemms)
    tc_out = C_.clone()
    capi.set_tuning(gemm_route=capi.ROUTE_INTEGER)
    ms_int = time_rotating(big_gemms)
    same = bool(torch.equal(tc_out, C_))
    capi.set_tuning()
    big_tops, int_tops = ops_big / (ms_big * 1e-3) / 1e12, ops_big / (ms_int * 1e-3) / 1e12
    traffic, traffic_source = captured_traffic("xnor_gemm_tcp_m512_n43264_k2304")
    out["roofline_large_batch"] = {
        "kernel": "xnor_gemm_tcp_kernel: persistent tcgen05 kind::mxf4 XNOR GEMM (bits widened to e2m1 +-1, results staged in shared memory and written by tensor stores; the library's own choice for this shape), M=512 N=64x676 K=2304", "bound": "tensor", "achieved": big_tops,
        "peak": umma_peak_tops, "unit": "TOP/s (binary ops, 2*M*N*K)", "frac": big_tops / umma_peak_tops,
        "traffic": traffic, "traffic_source": traffic_source, "algorithmic_bytes": alg_big,
        "peak_source": "measured in this run: back-to-back tcgen05.mma kind::mxf4 128x256x64 from resident shared memory",
        "kind_i8_rate": umma_i8_peak_tops, "frac_of_kind_i8_rate": big_tops / umma_i8_peak_tops,
        "vs_int_popc_peak": big_tops / popc_peak_tops, "ms": ms_big, "equals_integer_kernel": same,
        # the other roofline of the same launch: its 88.6 MB fp32 output against the copy rate (pure writes reach about 0.57 of it)
        "hbm_achieved_gbs": alg_big / (ms_big * 1e-3) / 1e9, "hbm_frac": alg_big / (ms_big * 1e-3) / 1e9 / hbm_peak,
    }
    # the longest rows of the three networks: tiny-yolo's last xnor layer at batch 256 (1024 filters, K = 9216)
    del As_, Bs_, Cs_
    Mk, Nk, Kk = 1024, 64 * 676, 9216
    ldk = Kk + (256 - Kk % 256)
    alg_k = (Mk + Nk) * ldk // 8 + 4 * Mk * Nk
    Ak = torch.randint(0, 256, (Mk, ldk // 8), dtype=torch.uint8, device=dev)
    Bk = torch.randint(0, 256, (Nk, ldk // 8), dtype=torch.uint8, device=dev)
    Ak[:, Kk // 8:] = 0
    Bk[:, Kk // 8:] = 0
    Aks = [Ak] + [Ak.clone() for _ in range(copies_for(alg_k) - 1)]
    Bks = [Bk] + [Bk.clone() for _ in range(len(Aks) - 1)]
    Cks = [torch.empty(Mk, Nk, device=dev) for _ in Aks]
    meank, biask = torch.rand(Mk, device=dev), torch.rand(Mk, device=dev)

    def long_gemm(i):
        def run():
            capi.check(lib.xnor_b200_gemm_bin_mean_transposed(Mk, Nk, Kk, Aks[i].data_ptr(), ldk, Bks[i].data_ptr(), ldk, Cks[i].data_ptr(), Nk,
                                                              meank.data_ptr(), biask.data_ptr(), 1, None, None, cur()), "gemm")
        return run
    ms_k = time_rotating([long_gemm(i) for i in range(len(Aks))])
    k_tops = 2.0 * Mk * Nk * Kk / (ms_k * 1e-3) / 1e12
    out["roofline_large_k"] = {
        "kernel": "xnor_gemm_tcp_kernel (persistent tcgen05 kind::mxf4 XNOR GEMM, the library's own choice), M=1024 N=64x676 K=9216", "bound": "tensor", "achieved": k_tops,
        "peak": umma_peak_tops, "unit": "TOP/s (binary ops, 2*M*N*K)", "frac": k_tops / umma_peak_tops, "traffic": None,
        "algorithmic_bytes": alg_k, "peak_source": out["roofline_large_batch"]["peak_source"],
        "frac_of_kind_i8_rate": k_tops / umma_i8_peak_tops, "vs_int_popc_peak": k_tops / popc_peak_tops, "ms": ms_k,
    }
    del Aks, Bks, Cks
    out["roofline_int_large_batch"] = {
        "kernel": "integer-pipe XNOR GEMM (tiled kernel, route pinned), M=512 N=64x676 K=2304", "bound": "int_popc", "achieved": int_tops,
        "peak": popc_peak_tops, "unit": "TOP/s (binary ops, 2*M*N*K)", "frac": int_tops / popc_peak_tops, "traffic": None,
        "algorithmic_bytes": alg_big, "peak_source": roofline["peak_source"], "ms": ms_int,
    }
    # The pack kernel of the same batch-64 layer (256 channels, 26x26, 3x3): HBM-bound, reported beside the batch-1 figure.
    lp = L.make_convolutional_layer(64, 26, 26, 256, 512, 3, 1, 1, capi.LEAKY, device=str(dev))
    bp_bytes = 64 * (4 * 256 * 26 * 26 + lp.geom.n_out * lp.new_lda // 8)
    n_bp = copies_for(bp_bytes)
    xp = torch.from_numpy(synth.bell(77, (64, 256, 26, 26))).to(dev)
    xps = [xp.clone() for _ in range(n_bp)]
    outps = [torch.empty(64 * lp.geom.n_out, lp.new_lda // 8, dtype=torch.uint8, device=dev) for _ in range(n_bp)]
    outp = outps[0]
    wordsp = torch.empty(lib.xnor_b200_pack_words_bytes(C.byref(lp.desc)), dtype=torch.uint8, device=dev)

    def big_pack(i):
        def run():
            capi.check(lib.xnor_b200_pack_input_staged(C.byref(lp.desc), xps[i].data_ptr(), wordsp.data_ptr(), outps[i].data_ptr(), cur()), "pack")
        return run

    def big_pack_single(i):
        def run():
            capi.check(lib.xnor_b200_pack_input(C.byref(lp.desc), xps[i].data_ptr(), outps[i].data_ptr(), cur()), "pack")
        return run
    ms_bp = time_rotating([big_pack_single(i) for i in range(n_bp)])
    single_out = outp.clone()
    capi.set_tuning(pack_two_pass=2)
    ms_bp2 = time_rotating([big_pack(i) for i in range(n_bp)])
    capi.set_tuning()
    traffic, traffic_source = captured_traffic("pack_input_words_b64_c256_26x26")
    out["roofline_pack_large_batch"] = {
        "kernel": "pack_input_words_kernel, batch 64, C=256, 26x26, 3x3",
        "bound": "hbm", "achieved": bp_bytes / (ms_bp * 1e-3) / 1e9,
        "peak": hbm_peak, "unit": "GB/s", "frac": bp_bytes / (ms_bp * 1e-3) / 1e9 / hbm_peak,
        "traffic": traffic, "traffic_source": traffic_source, "algorithmic_bytes": bp_bytes, "ms": ms_bp, "peak_source": hbm_source,
        "two_pass_ms": ms_bp2, "two_pass_frac": bp_bytes / (ms_bp2 * 1e-3) / 1e9 / hbm_peak,
        "two_pass_equals_single_kernel": bool(torch.equal(single_out, outp)),
    }
    # A larger map of the same kind (darknet53's 128-channel, 52x52 layers at batch 64), where rows allow 16-byte loads.
    lq = L.make_convolutional_layer(64, 52, 52, 128, 256, 3, 1, 1, capi.LEAKY, device=str(dev))
    bq_bytes = 64 * (4 * 128 * 52 * 52 + lq.geom.n_out * lq.new_lda // 8)
    n_bq = copies_for(bq_bytes)
    xq = torch.from_numpy(synth.bell(78, (64, 128, 52, 52))).to(dev)
    xqs = [xq] + [xq.clone() for _ in range(n_bq - 1)]
    outqs = [torch.empty(64 * lq.geom.n_out, lq.new_lda // 8, dtype=torch.uint8, device=dev) for _ in range(n_bq)]

    def pack52(i):
        def run():
            capi.check(lib.xnor_b200_pack_input(C.byref(lq.desc), xqs[i].data_ptr(), outqs[i].data_ptr(), cur()), "pack")
        return run
    ms_bq = time_rotating([pack52(i) for i in range(n_bq)])
    out["roofline_pack_52x52"] = {
        "kernel": "pack_input_words_kernel, batch 64, C=128, 52x52, 3x3", "bound": "hbm", "achieved": bq_bytes / (ms_bq * 1e-3) / 1e9,
        "peak": hbm_peak, "unit": "GB/s", "frac": bq_bytes / (ms_bq * 1e-3) / 1e9 / hbm_peak, "traffic": None,
        "algorithmic_bytes": bq_bytes, "ms": ms_bq, "peak_source": hbm_source,
    }
    del xqs, outqs, xps, outps
    out["gpu_reference"] = time_reference_gpu_kernels(time_rotating, copies_for, dev)
    if device_status(capi) != 0:
        raise SystemExit("bench: a bounded wait ran out in a roofline launch")
    return out, roofline


def time_reference_gpu_kernels(time_rotating, copies_for, dev):
    """The kernel to beat: the reference's OWN GPU xnor kernels (src-lib/im2col_kernels.cu, compiled unmodified for sm_100a
    into oracle/_ref/liboracle_refgpu.so) on BASELINE configuration 1, one image, called as forward_convolutional_layer_gpu
    calls them (repack_input_gpu_bin, im2col_ongpu, transpose_uint32_gpu, gemm_nn_custom_bin_mean_transposed_gpu = its wmma b1
    kernel), timed the same way as the library's own pack + GEMM on the same tensors.  None where that build is absent."""
    import torch
    import synth
    from darknet_b200 import capi
    from darknet_b200 import layer as L
    from oracle import binding
    so = getattr(binding, "REFGPU_SO", None)
    if not so or not os.path.exists(so):
        return None
    ref = C.CDLL(so)
    vp, ci = C.c_void_p, C.c_int
    ref.refgpu_xnor_chain.argtypes = [ci] * 7 + [vp] * 8 + [ci, ci, vp]
    c, h, w, n, ks = 256, 26, 26, 512, 3
    x, wt, b = synth.conv_case(4242, 1, c, h, w, n, ks)
    xg = torch.from_numpy(x).to(dev)
    l = L.make_convolutional_layer(1, h, w, c, n, ks, 1, 1, capi.LEAKY, device=str(dev))
    l.load_weights(torch.from_numpy(wt).to(dev), torch.from_numpy(b).to(dev))
    L.binary_align_weights(l)
    ours = L.forward_convolutional_layer_gpu(l, xg).clone()
    inv = L.make_convolutional_layer(1, h, w, c, n, ks, 1, 1, capi.LEAKY, device=str(dev))
    inv.load_weights(torch.from_numpy(wt).to(dev), torch.from_numpy(b).to(dev))
    L.binary_align_weights(inv, invert=True)              # the complemented layout Darknet's GPU build stores
    g = l.geom
    words = (g.bit_align * g.k)                            # the reference's own (generous) workspace size, in floats
    transposed_bytes = g.n_out * g.new_lda // 8 + 64
    sets = copies_for(4 * (xg.numel() + 2 * words + n * g.n_out) + transposed_bytes + inv.align_bit_weights_gpu.numel())
    xs = [xg.clone() for _ in range(sets)]
    align_ws = [torch.zeros(words, dtype=torch.float32, device=dev) for _ in range(sets)]
    workspace = [torch.zeros(words, dtype=torch.float32, device=dev) for _ in range(sets)]
    transposed = [torch.zeros(transposed_bytes, dtype=torch.uint8, device=dev) for _ in range(sets)]
    inv_w = [inv.align_bit_weights_gpu.clone() for _ in range(sets)]
    own_w = [l.align_bit_weights_gpu.clone() for _ in range(sets)]
    outs = [torch.empty(1, n, g.out_h, g.out_w, device=dev) for _ in range(sets)]
    scratch = [torch.zeros_like(l.scratch) for _ in range(sets)]
    out = outs[0]

    def cur() -> int:
        return torch.cuda.current_stream().cuda_stream

    def chain(i, gemm_only):
        def run():
            rc = ref.refgpu_xnor_chain(c, h, w, n, ks, 1, 1, xs[i].data_ptr(), align_ws[i].data_ptr(), workspace[i].data_ptr(), transposed[i].data_ptr(),
                                       inv_w[i].data_ptr(), inv.mean_arr_gpu.data_ptr(), inv.biases_gpu.data_ptr(), outs[i].data_ptr(),
                                       1, int(gemm_only), cur())
            if rc != 0:
                raise SystemExit(f"bench: the reference GPU kernels reported {rc}")
        return run

    ms_chain = time_rotating([chain(i, False) for i in range(sets)])
    ms_gemm = time_rotating([chain(i, True) for i in range(sets)])
    diff = float((out - ours).abs().max())

    def own_layer(i):
        def run():
            capi.check(capi.lib().xnor_b200_conv_forward(C.byref(l.desc), xs[i].data_ptr(), own_w[i].data_ptr(), l.mean_arr_gpu.data_ptr(),
                                                         l.biases_gpu.data_ptr(), outs[i].data_ptr(), None, None, scratch[i].data_ptr(),
                                                         scratch[i].numel(), cur()), "xnor_b200_conv_forward")
        return run

    def own_gemm(i):
        def run():
            capi.check(capi.lib().xnor_b200_gemm_bin_mean_transposed(n, g.n_out, g.k, own_w[i].data_ptr(), g.new_lda, scratch[i].data_ptr(),
                                                                     g.new_lda, outs[i].data_ptr(), g.n_out, l.mean_arr_gpu.data_ptr(), l.biases_gpu.data_ptr(),
                                                                     1, None, None, cur()), "gemm")
        return run
    ms_own = time_rotating([own_layer(i) for i in range(sets)])
    ms_own_gemm = time_rotating([own_gemm(i) for i in range(sets)])
    own_diff = float((out - ours).abs().max())
    ops = 2.0 * n * g.n_out * g.k
    return {
        "what": "BASELINE configuration 1 (3x3, 256 -> 512 filters, 26x26, leaky), one image; each side's calls rotate over copies of all "
                "buffers larger than twice the L2, one CUDA graph per sweep",
        "reference_kernels": "darknet src-lib/im2col_kernels.cu compiled unmodified for sm_100a (wmma b1 tensor kernel + its three input kernels)",
        "reference_layer_us": 1000.0 * ms_chain, "reference_gemm_us": 1000.0 * ms_gemm, "reference_gemm_tops": ops / (ms_gemm * 1e-3) / 1e12,
        "own_layer_us": 1000.0 * ms_own, "own_gemm_us": 1000.0 * ms_own_gemm, "own_gemm_tops": ops / (ms_own_gemm * 1e-3) / 1e12,
        "layer_speedup": ms_chain / ms_own, "gemm_speedup": ms_gemm / ms_own_gemm,
        "max_abs_difference_of_outputs": diff, "own_output_differs_from_layer_api_by": own_diff,
        "note": "the reference computes count*mean+bias with one fused multiply-add on the GPU, this library with the CPU path's two roundings, hence a last-bit difference",
    }


# ---- single kernels (profiler captures, quick timings) ---------------------------------------------

YOLOV3_TINY_GEMMS = [(32, 43264, 144), (64, 10816, 288), (128, 2704, 576), (256, 676, 1152), (512, 169, 2304), (1024, 169, 4608),
                     (256, 169, 1024), (128, 169, 256), (256, 676, 3456)]
FCONV_CASES = [(1, 256, 13, 13, 512, 3, 1), (1, 512, 13, 13, 255, 1, 0), (1, 256, 26, 26, 255, 1, 0)]


def run_kernel(args) -> None:
    """One kernel of libxnor_b200.so on random operands, `reps` calls each between two CUDA events; prints the median
    (not meaningful under a profiler).  Ends with a synchronize and a device-status check."""
    import torch
    from darknet_b200 import capi
    from darknet_b200 import layer as L
    if not torch.cuda.is_available():
        raise SystemExit("bench.py --kernel needs a CUDA device")
    lib = capi.lib()
    capi.set_tuning(gemm_route=ROUTES[args.route], tc_kernel=args.tc_kernel, pack_ctas_per_sm=args.pack_ctas_per_sm)

    def stream() -> int:
        return torch.cuda.current_stream().cuda_stream

    side = torch.cuda.Stream()

    def copies_for(set_bytes: int) -> int:
        return max(2, -(-int(2.2 * L2_BYTES) // max(int(set_bytes), 1)))

    def timed(calls, reps: int) -> float:
        """Median microseconds of ONE of `calls`, which do the same work on separate copies of their buffers (together more
        than twice the L2).  A whole rotation is captured into one CUDA graph and timed between two events, so neither host
        launch overhead nor the cost of an event pair ends up in a call's figure.  With --no-graph (profiler captures) the
        calls are launched directly and the figure includes the host."""
        ts = []
        if args.no_graph:
            for r in range(reps):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                calls[r % len(calls)]()
                b.record()
                torch.cuda.synchronize()
                ts.append(a.elapsed_time(b) * 1000.0)
            return sorted(ts)[len(ts) // 2]
        torch.cuda.synchronize()
        with torch.cuda.stream(side):
            for fn in calls:
                fn()
            side.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                for fn in calls:
                    fn()
            evs = []
            for _ in range(2):
                g.replay()
            for _ in range(reps):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(side)
                g.replay()
                b.record(side)
                evs.append((a, b))
            side.synchronize()
        ts = [a.elapsed_time(b) * 1000.0 / len(calls) for a, b in evs]
        return sorted(ts)[len(ts) // 2]

    def gemm_calls(M, N, K, shortcut, copies=None):
        lda = K + (256 - K % 256)
        per_set = (M + N) * lda // 8 + 4 * M * N * (3 if shortcut else 1)
        calls, keep = [], []
        for _ in range(copies or copies_for(per_set)):
            A = torch.randint(0, 256, (M, lda // 8), dtype=torch.uint8, device="cuda")
            B = torch.randint(0, 256, (N, lda // 8), dtype=torch.uint8, device="cuda")
            A[:, K // 8:] = 0
            B[:, K // 8:] = 0
            out = torch.empty(M, N, device="cuda")
            mean, bias = torch.rand(M, device="cuda"), torch.rand(M, device="cuda")
            sc_in = torch.randn(M, N, device="cuda") if shortcut else None
            sc_out = torch.empty(M, N, device="cuda") if shortcut else None
            bufs = (A, B, out, mean, bias, sc_in, sc_out)
            keep.append(bufs)

            def call(bufs=bufs):
                A, B, out, mean, bias, sc_in, sc_out = bufs
                capi.check(lib.xnor_b200_gemm_bin_mean_transposed(
                    M, N, K, A.data_ptr(), lda, B.data_ptr(), lda, out.data_ptr(), N, mean.data_ptr(), bias.data_ptr(), 1,
                    sc_in.data_ptr() if shortcut else None, sc_out.data_ptr() if shortcut else None, stream()), "xnor_b200_gemm_bin_mean_transposed")
            calls.append(call)
        return calls, keep

    if args.kernel == "gemm":
        M, N, K = args.shape
        calls, _keep = gemm_calls(M, N, K, args.shortcut)
        us = timed(calls, args.reps)
        print(f"gemm M={M} N={N} K={K} route={args.route} shortcut={int(args.shortcut)}: {us:.1f} us/call, {2.0 * M * N * K / us / 1e6:.1f} T binary ops/s")
    elif args.kernel == "gemms":
        keep = []
        for _ in range(2):
            for (M, N, K) in YOLOV3_TINY_GEMMS:
                calls, k = gemm_calls(M, N, K, False, copies=1)
                keep.append(k)
                calls[0]()
        torch.cuda.synchronize()
        print("ok")
    elif args.kernel == "pack":
        batch, c, h, w, n, ks = args.shape
        l = L.make_convolutional_layer(batch, h, w, c, n, ks, 1, ks // 2, capi.LINEAR)
        rows_bytes = batch * l.geom.n_out * l.new_lda // 8
        moved = batch * c * h * w * 4 + rows_bytes
        xs = [torch.randn(batch, c, h, w, device="cuda") for _ in range(copies_for(moved))]
        xs = [xs[0]] + [xs[0].clone() for _ in xs[1:]]
        outs = [torch.empty(batch * l.geom.n_out, l.new_lda // 8, dtype=torch.uint8, device="cuda") for _ in xs]

        def single(i):
            return lambda: capi.check(lib.xnor_b200_pack_input(C.byref(l.desc), xs[i].data_ptr(), outs[i].data_ptr(), stream()), "xnor_b200_pack_input")
        us = timed([single(i) for i in range(len(xs))], args.reps)
        print(f"pack b={batch} c={c} {h}x{w} ks={ks}: {us:.1f} us/call, {moved / us / 1e3:.0f} GB/s")
        if c % 32 == 0:
            want = outs[-1].clone()
            words = torch.empty(lib.xnor_b200_pack_words_bytes(C.byref(l.desc)), dtype=torch.uint8, device="cuda")
            capi.set_tuning(pack_two_pass=2, pack_ctas_per_sm=args.pack_ctas_per_sm)

            def staged(i):
                return lambda: capi.check(lib.xnor_b200_pack_input_staged(C.byref(l.desc), xs[i].data_ptr(), words.data_ptr(), outs[i].data_ptr(),
                                                                          stream()), "xnor_b200_pack_input_staged")
            us = timed([staged(i) for i in range(len(xs))], args.reps)
            capi.set_tuning()
            print(f"pack b={batch} c={c} {h}x{w} ks={ks} in two passes: {us:.1f} us/call, {moved / us / 1e3:.0f} GB/s, "
                  f"equal={bool(torch.equal(want, outs[-1]))}")
    elif args.kernel == "layer":
        # one xnor layer's GEMM on an operand packed beforehand: the fp32 tensor, or (--sum-only) only the sum with a shortcut
        # operand and the sum's sign words, as darknet53's residual blocks ask for it
        batch, c, h, w, n, ks = args.shape[:6]
        stride = args.shape[6] if len(args.shape) > 6 else 1
        wt = torch.randn(n, c * ks * ks, device="cuda") * 0.05
        bias = torch.randn(n, device="cuda") * 0.3
        x = torch.randn(batch, c, h, w, device="cuda")
        probe = L.make_convolutional_layer(batch, h, w, c, n, ks, stride, ks // 2, capi.LEAKY)
        out_bytes = 4 * batch * n * probe.geom.n_out
        moved = batch * probe.geom.n_out * probe.new_lda // 8 + out_bytes * (2 if args.sum_only else 1)
        layers = []
        for _ in range(copies_for(moved)):
            l = L.make_convolutional_layer(batch, h, w, c, n, ks, stride, ks // 2, capi.LEAKY)
            l.load_weights(wt, bias)
            L.binary_align_weights(l)
            op = L.pack_input(l, x)
            l.scratch[:op.numel()].copy_(op.view(-1))
            if args.sum_only:
                l.bin_conv_shortcut_in_gpu = torch.randn(batch, n, probe.geom.out_h, probe.geom.out_w, device="cuda")
                l.bin_conv_shortcut_out_gpu = torch.empty_like(l.bin_conv_shortcut_in_gpu)
            layers.append(l)

        def layer_call(l):
            if args.sum_only:
                return lambda: L.forward_convolutional_layer_io(l, packed=True, shortcut_only=True, shortcut_signs=True)
            return lambda: L.forward_convolutional_layer_io(l, packed=True, want_output=True)
        us = timed([layer_call(l) for l in layers], args.reps)
        print(f"layer b={batch} c={c} {h}x{w} n={n} ks={ks} stride={stride} route={args.route} sum_only={int(args.sum_only)}: {us:.1f} us/call, "
              f"{moved / us / 1e3:.0f} GB/s of operand + fp32 bytes")
    else:
        b, c, h, w, n, ks, leaky = FCONV_CASES[args.shape[0]]
        x = torch.randn(b, c, h, w, device="cuda")
        wt = torch.randn(n, c, ks, ks, device="cuda") * 0.05
        bias = torch.randn(n, device="cuda")
        d = capi.ConvDesc(b, c, h, w, n, ks, 1, ks // 2, capi.LEAKY if leaky else capi.LINEAR)
        blocked = torch.empty(lib.xnor_b200_float_conv_map_weights_bytes(C.byref(d)) // 4, device="cuda")
        out = torch.empty(b, n, h, w, device="cuda")
        capi.check(lib.xnor_b200_float_conv_map_prepare(C.byref(d), wt.data_ptr(), blocked.data_ptr(), stream()), "xnor_b200_float_conv_map_prepare")

        def call():
            capi.check(lib.xnor_b200_float_conv_map(C.byref(d), x.data_ptr(), blocked.data_ptr(), bias.data_ptr(), out.data_ptr(), stream()),
                       "xnor_b200_float_conv_map")
        us = timed([call], args.reps)
        print(f"fconv {FCONV_CASES[args.shape[0]]}: {us:.1f} us/call (one buffer set: L2-warm)")
    st = device_status(capi)
    if st != 0:
        raise SystemExit(f"device status {st}: a bounded wait ran out")


def main() -> None:
    args = parse_args()
    if args.kernel is not None:
        run_kernel(args)
    elif args.impl == "reference":
        run_reference_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
