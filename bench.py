#!/usr/bin/env python
"""Benchmark of the xnor conv path on B200: yolov3-tiny_xnor forward at 416x416, batch 1 per GPU.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One "step" is one forward pass of the network over one batch of seeded synthetic input with seeded
random weights (no dataset or checkpoint is involved).  Every xnor=1 convolution runs through
libxnor_b200.so; the float layers around the path run through cuDNN/ATen as they run through cuDNN in
Darknet.  The forward is captured once into a CUDA graph and replayed.

Printed JSON (one line, rank 0):
  value      images/s, inputs resident in HBM, per-step CUDA-event time (max over ranks), L2 flushed
             between steps
  e2e        images/s through the same call with the input copied from pinned host memory and the head
             outputs copied back inside the timed region
  roofline   the XNOR GEMM launches of one forward, timed alone with CUDA events on their stream, against
             the integer XOR+POPC+ADD issue rate measured on the same GPU in the same run
  cpu_baseline  the reference's own CPU xnor code (oracle/_ref) on the same layer shapes, host cores

--impl reference times only that CPU code (xnor layers of the same network) and prints its own line.
With N > 1 (torchrun) every rank runs an independent replica on its GPU: replicas only, no collective on
the data path; NCCL is used for the barrier and the max over ranks.
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

WORKLOAD = "yolov3-tiny_xnor forward, 416x416x3 fp32 input U[0,1), batch 1 per GPU, seeded random weights"
METRIC = "images/s yolov3-tiny_xnor@416"
L2_FLUSH_BYTES = 256 << 20


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=500)
    ap.add_argument("--warmup", type=int, default=50)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--batch", type=int, default=1, help="images per GPU per step (the metric is quoted at 1)")
    ap.add_argument("--cpu-baseline-seconds", type=float, default=12.0)
    ap.add_argument("--workload", default="yolov3-tiny_xnor", choices=["yolov3-tiny_xnor", "tiny-yolo_xnor", "darknet53_448_xnor"],
                    help="network to run; the default is the configuration the metric is quoted on, the others are the "
                         "batched BASELINE configurations (use with --batch)")
    return ap.parse_args()


# ---- CPU reference arm ---------------------------------------------------------------------------

def xnor_layer_table():
    import torch  # noqa: F401  (network.py imports torch; CPU only here)
    from darknet_b200 import cfgs, network
    with tempfile.TemporaryDirectory() as td:
        p = os.path.join(td, "net.cfg")
        with open(p, "w") as fh:
            fh.write(cfgs.yolov3_tiny_xnor_cfg())
        net = network.parse_network_cfg(p, 1, "cpu")
    # bin_output layers lose their activation at load (calculate_binary_weights)
    rows = network.xnor_layer_shapes(net)
    for r, l in zip(rows, [l for l in net.layers if l.type == "convolutional" and l.xnor]):
        r["leaky"] = int(l.activation == "leaky" and not l.use_bin_output)
    return rows


class CpuReference:
    """The reference's CPU xnor forward (oracle/_ref: its own sources compiled unmodified) over the xnor layers
    of the workload; where that build is absent, the plain-C restatement.  Built once, then timed."""

    def __init__(self, threads: int | None = None) -> None:
        import synth
        from oracle.binding import Port, Ref
        self.rows = xnor_layer_table()
        self.cores = threads or os.cpu_count() or 1
        if Ref.available():
            ref = Ref()
            ref.set_gpu_index(-1)
            ref.set_num_threads(self.cores)
            self.kind = "reference"
            self.layers = []
            for i, r in enumerate(self.rows):
                x, wt, b = synth.conv_case(900 + i, 1, r["c"], r["h"], r["w"], r["n"], r["size"])
                self.layers.append((ref.layer((r["c"], r["h"], r["w"]), wt, b, r["stride"], r["pad"], bool(r["leaky"])), x[0]))
            self._one = lambda: [lay.forward(x) for lay, x in self.layers]
        else:
            port = Port()
            self.kind = "port"
            cases = [(synth.conv_case(900 + i, 1, r["c"], r["h"], r["w"], r["n"], r["size"]), r) for i, r in enumerate(self.rows)]
            self._one = lambda: [port.conv_forward(x, wt, b, r["stride"], r["pad"], r["leaky"]) for (x, wt, b), r in cases]
        self._one()  # warm-up (page-in, OpenMP pool)

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
        return (f"{images} images x {len(self.rows)} xnor layers of yolov3-tiny_xnor@416 (float layers excluded), "
                f"{seconds:.1f} s, {self.cores} threads")


def time_cpu_reference(budget_s: float):
    cpu = CpuReference()
    n = cpu.images_for(budget_s)
    el = cpu.run(n)
    return n / el, cpu.kind, cpu.cores, cpu.describe(n, el)


def run_reference_arm(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cpu = CpuReference()
    per_step = max(0.2, min(2.0, 150.0 / max(args.steps + args.warmup, 1)))
    n = cpu.images_for(per_step)        # images per step: a bounded sample of the workload
    for _ in range(args.warmup):
        cpu.run(n)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu.run(n)
    el = time.perf_counter() - t0
    value = n * args.steps / el
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "images/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1000.0 * el / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "u32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "scope": "xnor conv layers only (the path), reference CPU code on host cores",
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


def run_gpu_arm(args) -> None:
    import torch
    import torch.distributed as dist
    import synth
    from darknet_b200 import capi, cfgs, network, replicas
    from darknet_b200 import layer as L

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

    batch = args.batch
    with tempfile.TemporaryDirectory() as td:
        cfg_path, w_path = os.path.join(td, "yolov3-tiny_xnor.cfg"), os.path.join(td, "synthetic.weights")
        with open(cfg_path, "w") as fh:
            fh.write(cfgs.CFGS[args.workload]())
        net0 = network.parse_network_cfg(cfg_path, batch, "cpu")
        network.write_synthetic_weights(net0, w_path, seed=1)
        net = network.load_network_custom(cfg_path, w_path, batch, str(dev))
    rows = network.xnor_layer_shapes(net)
    binops_per_image = sum(r["binops"] for r in rows)

    default_workload = (args.workload == "yolov3-tiny_xnor")
    workload_text = WORKLOAD if default_workload and batch == 1 else \
        f"{args.workload} forward, {net.h}x{net.w}x3 fp32 input U[0,1), batch {batch} per GPU, seeded random weights"
    metric_text = METRIC if default_workload else f"images/s {args.workload}@{net.h}"
    x_host = torch.from_numpy(synth.uniform01(1 + rank, (batch, 3, net.h, net.w))).pin_memory()
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
    # the end-to-end step as one graph: input copy from pinned memory, forward, every head copied to pinned memory on
    # the stream that produced it
    graph_e2e = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph_e2e, stream=stream):
        x_dev.copy_(x_host, non_blocking=True)
        heads_e2e = network.forward_network_gpu(net, x_dev, head_host)
    h2d_bytes = x_host.numel() * 4
    d2h_bytes = sum(h.numel() * 4 for h in heads)

    def barrier():
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def timed_steps(n_steps: int, end_to_end: bool) -> float:
        """Returns total milliseconds of n_steps forwards (sum of per-step CUDA-event intervals; the L2 flush
        between steps sits outside the intervals)."""
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n_steps)]
        with torch.cuda.stream(stream):
            for a, b in evs:
                flush.fill_(1)
                a.record(stream)
                if end_to_end:
                    graph_e2e.replay()
                else:
                    graph.replay()
                b.record(stream)
        stream.synchronize()
        return float(sum(a.elapsed_time(b) for a, b in evs))

    def max_over_ranks(ms: float) -> float:
        return replicas.max_over_ranks(ms, dev)

    sampler = ClockSampler(local) if rank == 0 else None
    timed_steps(args.warmup, False)
    barrier()
    ms_total = timed_steps(args.steps, False)
    barrier()
    ms_total = max_over_ranks(ms_total)
    timed_steps(max(3, args.warmup // 4), True)
    barrier()
    ms_e2e = timed_steps(args.steps, True)
    barrier()
    ms_e2e = max_over_ranks(ms_e2e)
    for hh, hd in zip(head_host, heads):               # what the end-to-end steps left in pinned host memory = the device-resident forward
        if not torch.equal(hh, hd.cpu()):
            raise SystemExit("bench: host copy of a head differs from the device tensor")
    clocks = sampler.stop() if sampler else None

    value = world * batch * args.steps / (ms_total * 1e-3)
    e2e_value = world * batch * args.steps / (ms_e2e * 1e-3)

    # ---- roofline of the dominant kernel (XNOR GEMM), rank 0 only ----
    roofline = pack_roofline = large_roofline = large_pack_roofline = cpu_baseline = None
    if rank == 0 and default_workload:
        lib = capi.lib()
        xl_layers = [l.xnor_layer for l in net.layers if l.type == "convolutional" and l.xnor]
        inputs = [torch.from_numpy(synth.bell(50 + i, (batch, xl.c, xl.h, xl.w))).to(dev) for i, xl in enumerate(xl_layers)]
        packed = [L.pack_input(xl, xi) for xl, xi in zip(xl_layers, inputs)]
        torch.cuda.synchronize(dev)
        reps = 50

        def time_launches(fn) -> float:
            """Average ms of one pass over all xnor layers: the launches are captured into a CUDA graph (so host
            launch overhead is not what gets timed) and replayed with the L2 flushed before each pass."""
            with torch.cuda.stream(stream):
                fn()
            stream.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                fn()
            evs = []
            with torch.cuda.stream(stream):
                for _ in range(5):
                    g.replay()
                for _ in range(reps):
                    flush.fill_(1)
                    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    a.record(stream)
                    g.replay()
                    b.record(stream)
                    evs.append((a, b))
            stream.synchronize()
            return sum(a.elapsed_time(b) for a, b in evs) / reps

        def all_gemms():
            for xl, pk in zip(xl_layers, packed):
                g = xl.geom
                capi.check(lib.xnor_b200_gemm_bin_mean_transposed(
                    xl.n, batch * g.n_out, g.k, xl.align_bit_weights_gpu.data_ptr(), g.new_lda, pk.data_ptr(), g.new_lda,
                    xl.output_gpu.data_ptr(), batch * g.n_out, xl.mean_arr_gpu.data_ptr(), xl.biases_gpu.data_ptr(),
                    int(xl.activation == capi.LEAKY), None, None, torch.cuda.current_stream().cuda_stream), "gemm")

        def all_packs():
            for xl, xi, pk in zip(xl_layers, inputs, packed):
                capi.check(lib.xnor_b200_pack_input(C.byref(xl.desc), xi.data_ptr(), pk.data_ptr(), torch.cuda.current_stream().cuda_stream), "pack")

        ms_gemm = time_launches(all_gemms)
        ms_pack = time_launches(all_packs)
        g_, m_ = C.c_double(), C.c_double()
        capi.check(lib.xnor_b200_measure_popc_peak(20000, C.byref(g_), C.byref(m_)), "popc peak")
        popc_peak_tops = g_.value / 1e3
        capi.check(lib.xnor_b200_measure_bmma_peak(2000, C.byref(g_), C.byref(m_)), "bmma peak")
        bmma_peak_tops = g_.value / 1e3
        achieved = binops_per_image * batch / (ms_gemm * 1e-3) / 1e12
        roofline = {
            "kernel": "xnor_gemm_kernel (9 launches = the xnor layers of one forward, stand-alone calls with fp32 epilogue)",
            "bound": "int_popc", "achieved": achieved, "peak": popc_peak_tops, "unit": "TOP/s (binary ops, 2*M*N*K)",
            # dram__bytes_read + dram__bytes_write summed over the 9 launches of one forward (batch 1), one ncu capture:
            # profiles/xnor_gemm_kernels_b1_dram_traffic.md.  Algorithmic bytes = packed operands read once + fp32 outputs.
            "frac": achieved / popc_peak_tops, "traffic": 4.36e6 if batch == 1 else None,
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
        pack_gbs = pack_bytes / (ms_pack * 1e-3) / 1e9
        pack_roofline = {
            "kernel": "pack_input_*_kernel (9 launches: every xnor layer's stand-alone xnor_b200_pack_input; the linked forward replaces most of them by sign sinks)", "bound": "hbm", "achieved": pack_gbs, "peak": hbm_peak, "unit": "GB/s",
            "frac": pack_gbs / hbm_peak, "traffic": None, "ms_per_forward": ms_pack,
            "peak_source": "MEASURED_PEAKS.json (of measured)" if peaks else "fallback 6650 GB/s (of fallback)",
        }
        # The same GEMM entry point on a batch-64 layer (BASELINE config 1 shape: 256 -> 512 filters, 26x26, 3x3), where the
        # library switches to the tcgen05 kernel: reported beside the headline because batch-1 launches are latency-bound.
        capi.check(lib.xnor_b200_measure_umma_i8_peak(4000, C.byref(g_), C.byref(m_)), "umma peak")
        umma_peak_tops = g_.value / 1e3
        M_, N_, K_ = 512, 64 * 676, 2304
        lda_ = K_ + (256 - K_ % 256)
        A_ = torch.randint(0, 256, (M_, lda_ // 8), dtype=torch.uint8, device=dev)
        B_ = torch.randint(0, 256, (N_, lda_ // 8), dtype=torch.uint8, device=dev)
        A_[:, K_ // 8:] = 0
        B_[:, K_ // 8:] = 0
        C_ = torch.empty(M_, N_, device=dev)
        mean_ = torch.rand(M_, device=dev)
        bias_ = torch.rand(M_, device=dev)

        def big_gemm():
            capi.check(lib.xnor_b200_gemm_bin_mean_transposed(M_, N_, K_, A_.data_ptr(), lda_, B_.data_ptr(), lda_, C_.data_ptr(), N_,
                                                              mean_.data_ptr(), bias_.data_ptr(), 1, None, None,
                                                              torch.cuda.current_stream().cuda_stream), "gemm")
        ms_big = time_launches(big_gemm)
        big_tops = 2.0 * M_ * N_ * K_ / (ms_big * 1e-3) / 1e12
        large_roofline = {
            "kernel": "xnor_gemm_tc_kernel<256> (tcgen05 kind::i8), M=512 N=64x676 K=2304", "bound": "tensor", "achieved": big_tops,
            "peak": umma_peak_tops, "unit": "TOP/s (binary ops, 2*M*N*K)", "frac": big_tops / umma_peak_tops,
            # dram read + write of one launch of this shape, ncu capture summarised in profiles/xnor_gemm_tc_kernel_m512_n43264_k2304.md
            "traffic": 44.41e6,
            "peak_source": "measured in this run: back-to-back tcgen05.mma kind::i8 128x256x32 from resident shared memory",
            "vs_int_popc_peak": big_tops / popc_peak_tops, "ms": ms_big,
        }
        # The pack kernel of the same batch-64 layer (256 channels, 26x26, 3x3): HBM-bound, reported beside the batch-1 figure.
        from darknet_b200 import layer as L2
        lp = L2.make_convolutional_layer(64, 26, 26, 256, 512, 3, 1, 1, capi.LEAKY, device=str(dev))
        xp = torch.from_numpy(synth.bell(77, (64, 256, 26, 26))).to(dev)
        outp = torch.empty(64 * lp.geom.n_out, lp.new_lda // 8, dtype=torch.uint8, device=dev)

        def big_pack():
            capi.check(lib.xnor_b200_pack_input(C.byref(lp.desc), xp.data_ptr(), outp.data_ptr(), torch.cuda.current_stream().cuda_stream), "pack")
        ms_bp = time_launches(big_pack)
        bp_bytes = 64 * (4 * 256 * 26 * 26 + lp.geom.n_out * lp.new_lda // 8)
        large_pack_roofline = {
            "kernel": "pack_input_words_kernel<2,1,0>, batch 64, C=256, 26x26, 3x3", "bound": "hbm", "achieved": bp_bytes / (ms_bp * 1e-3) / 1e9,
            "peak": hbm_peak, "unit": "GB/s", "frac": bp_bytes / (ms_bp * 1e-3) / 1e9 / hbm_peak,
            # dram read + write of one launch, ncu capture summarised in profiles/pack_input_words_kernel_b64_c256_26x26.md
            "traffic": 44.41e6, "ms": ms_bp,
            "peak_source": pack_roofline["peak_source"],
        }
        if world == 1:
            ips, kind, cores, sample = time_cpu_reference(args.cpu_baseline_seconds)
            cpu_baseline = {"value": ips, "unit": "images/s", "cores": cores, "kind": kind, "sample": sample}

    if rank == 0:
        line = {
            "metric": metric_text, "value": value, "unit": "images/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_total / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "u32", "data": "synthetic",
            "config": {"workload": workload_text, "global_batch": world * batch, "folded_maxpools": net.folded_maxpools, "sign_sinks": net.sink_links, "sign_links": net.sign_links,
                       "side_branch": any(l.branch_start for l in net.layers), "parallelism": f"replicas x{world} (no collective)",
                       "l2": "256 MiB buffer written between timed steps", "timing": "per-step CUDA events on the launch stream, CUDA graph replay",
                       "float_layers": "this library's fp32 kernels at small batch (first conv + pool + sign, small-map convs with the yolo activation), cuDNN/ATen otherwise",
                       "xnor_binops_per_image": binops_per_image},
            "xnor_gemm_tops": roofline["achieved"] if roofline else None,
            "roofline": roofline, "roofline_pack": pack_roofline, "roofline_large_batch": large_roofline, "roofline_pack_large_batch": large_pack_roofline,
            "cpu_baseline": cpu_baseline,
            "e2e": {"value": e2e_value, "unit": "images/s", "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": d2h_bytes,
                    "ms_per_step": ms_e2e / args.steps},
            "gpu_launches": args.steps * network.own_launches_per_forward(net),
            "clocks": clocks,
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def main() -> None:
    args = parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
