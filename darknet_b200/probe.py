"""Runs one kernel of libxnor_b200.so a few times on random operands -- the small driver the profiler captures are
made with (``ncu ... python -m darknet_b200.probe gemm 512 43264 2304 3``) and a quick way to time a shape.

    python -m darknet_b200.probe gemm  M N K REPS [--shortcut]       xnor_b200_gemm_bin_mean_transposed, leaky + bias
    python -m darknet_b200.probe gemms                               the nine GEMM shapes of a batch-1 yolov3-tiny forward, twice
    python -m darknet_b200.probe pack  BATCH C H W N KS REPS         xnor_b200_pack_input (stride 1, pad KS/2)
    python -m darknet_b200.probe fconv CASE                          xnor_b200_float_conv_map on one of three yolov3-tiny shapes

XNOR_B200_GEMM_TC=1 / =0 in the environment pins the GEMM to the tensor-core / integer kernel.  Every run ends with a
synchronize and prints the median time per call measured with CUDA events (not meaningful under a profiler).
"""
from __future__ import annotations

import argparse
import ctypes as C

import torch

from . import capi, layer as L

YOLOV3_TINY_GEMMS = [(32, 43264, 144), (64, 10816, 288), (128, 2704, 576), (256, 676, 1152), (512, 169, 2304), (1024, 169, 4608),
                     (256, 169, 1024), (128, 169, 256), (256, 676, 3456)]
FCONV_CASES = [(1, 256, 13, 13, 512, 3, 1), (1, 512, 13, 13, 255, 1, 0), (1, 256, 26, 26, 255, 1, 0)]


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _timed(fn, reps: int) -> float:
    """Median microseconds per call over `reps` calls, each between two events."""
    ts = []
    for _ in range(reps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b) * 1000.0)
    return sorted(ts)[len(ts) // 2]


def _gemm_call(M: int, N: int, K: int, shortcut: bool):
    lda = K + (256 - K % 256)
    A = torch.randint(0, 256, (M, lda // 8), dtype=torch.uint8, device="cuda")
    B = torch.randint(0, 256, (N, lda // 8), dtype=torch.uint8, device="cuda")
    out = torch.empty(M, N, device="cuda")
    mean, bias = torch.rand(M, device="cuda"), torch.rand(M, device="cuda")
    sc_in = torch.randn(M, N, device="cuda") if shortcut else None
    sc_out = torch.empty(M, N, device="cuda") if shortcut else None
    keep = (A, B, out, mean, bias, sc_in, sc_out)

    def call():
        capi.check(capi.lib().xnor_b200_gemm_bin_mean_transposed(
            M, N, K, A.data_ptr(), lda, B.data_ptr(), lda, out.data_ptr(), N, mean.data_ptr(), bias.data_ptr(), 1,
            sc_in.data_ptr() if shortcut else None, sc_out.data_ptr() if shortcut else None, _stream()), "xnor_b200_gemm_bin_mean_transposed")
    return call, keep


def gemm(args) -> None:
    call, _keep = _gemm_call(args.M, args.N, args.K, args.shortcut)
    us = _timed(call, args.reps)
    ops = 2.0 * args.M * args.N * args.K
    print(f"gemm M={args.M} N={args.N} K={args.K} shortcut={int(args.shortcut)}: {us:.1f} us/call, {ops / us / 1e6:.1f} T binary ops/s")


def gemms(_args) -> None:
    keep = []
    for _ in range(2):
        for (M, N, K) in YOLOV3_TINY_GEMMS:
            call, k = _gemm_call(M, N, K, False)
            keep.append(k)
            call()
    torch.cuda.synchronize()
    print("ok")


def pack(args) -> None:
    l = L.make_convolutional_layer(args.batch, args.h, args.w, args.c, args.n, args.ks, 1, args.ks // 2, capi.LINEAR)
    x = torch.randn(args.batch, args.c, args.h, args.w, device="cuda")
    out = torch.empty(args.batch * l.geom.n_out, l.new_lda // 8, dtype=torch.uint8, device="cuda")

    def call():
        capi.check(capi.lib().xnor_b200_pack_input(C.byref(l.desc), x.data_ptr(), out.data_ptr(), _stream()), "xnor_b200_pack_input")
    us = _timed(call, args.reps)
    moved = x.numel() * 4 + out.numel()
    print(f"pack b={args.batch} c={args.c} {args.h}x{args.w} ks={args.ks}: {us:.1f} us/call, {moved / us / 1e3:.0f} GB/s")


def fconv(args) -> None:
    b, c, h, w, n, ks, leaky = FCONV_CASES[args.case]
    lib = capi.lib()
    x = torch.randn(b, c, h, w, device="cuda")
    wt = torch.randn(n, c, ks, ks, device="cuda") * 0.05
    bias = torch.randn(n, device="cuda")
    d = capi.ConvDesc(b, c, h, w, n, ks, 1, ks // 2, capi.LEAKY if leaky else capi.LINEAR)
    blocked = torch.empty(lib.xnor_b200_float_conv_map_weights_bytes(C.byref(d)) // 4, device="cuda")
    out = torch.empty(b, n, h, w, device="cuda")
    capi.check(lib.xnor_b200_float_conv_map_prepare(C.byref(d), wt.data_ptr(), blocked.data_ptr(), _stream()), "xnor_b200_float_conv_map_prepare")

    def call():
        capi.check(lib.xnor_b200_float_conv_map(C.byref(d), x.data_ptr(), blocked.data_ptr(), bias.data_ptr(), out.data_ptr(), _stream()),
                   "xnor_b200_float_conv_map")
    us = _timed(call, 5)
    print(f"fconv {FCONV_CASES[args.case]}: {us:.1f} us/call")


def main() -> None:
    ap = argparse.ArgumentParser(prog="python -m darknet_b200.probe", description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="cmd", required=True)
    g = sub.add_parser("gemm")
    for name in ("M", "N", "K", "reps"):
        g.add_argument(name, type=int)
    g.add_argument("--shortcut", action="store_true")
    g.set_defaults(fn=gemm)
    sub.add_parser("gemms").set_defaults(fn=gemms)
    p = sub.add_parser("pack")
    for name in ("batch", "c", "h", "w", "n", "ks", "reps"):
        p.add_argument(name, type=int)
    p.set_defaults(fn=pack)
    f = sub.add_parser("fconv")
    f.add_argument("case", type=int, choices=range(len(FCONV_CASES)))
    f.set_defaults(fn=fconv)
    args = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("darknet_b200.probe needs a GPU")
    args.fn(args)


if __name__ == "__main__":
    main()
