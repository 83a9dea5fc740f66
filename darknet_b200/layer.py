"""Host-side mirror of Darknet's xnor convolutional layer life cycle, over the C ABI.

The names follow the reference so that tests read like its call sequence:

    l = make_convolutional_layer(batch, h, w, c, n, size, stride, pad, activation, xnor=1)
    l.load_weights(weights, biases)          # what load_convolutional_weights + fuse_conv_batchnorm leave
    binary_align_weights(l)                  # src-lib/convolutional_layer.cpp:1339
    forward_convolutional_layer_gpu(l, x)    # src-lib/convolutional_kernels.cu:181 (xnor branch)

torch is used for device memory and the current stream only; every computation is a call into
libxnor_b200.so.  Nothing here has a CPU path.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import capi


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


class ConvolutionalLayer:
    """The Darknet::Layer fields the xnor path touches (src-lib/darknet_layers.hpp:39-83, :250-261)."""

    def __init__(self, batch, h, w, c, n, size, stride, pad, activation, device="cuda:0") -> None:
        self.desc = capi.ConvDesc(batch, c, h, w, n, size, stride, pad, activation)
        g = capi.geometry(self.desc)
        self.batch, self.h, self.w, self.c, self.n = batch, h, w, c, n
        self.size, self.stride, self.pad, self.activation = size, stride, pad, activation
        self.xnor = 1
        self.out_h, self.out_w, self.out_c = g.out_h, g.out_w, n
        self.outputs = n * g.n_out
        self.lda_align = 256
        self.new_lda = g.new_lda
        self.bit_align = g.bit_align
        self.geom = g
        self.device = torch.device(device)
        self.weights_gpu = torch.zeros(n, c * size * size, dtype=torch.float32, device=self.device)
        self.biases_gpu = torch.zeros(n, dtype=torch.float32, device=self.device)
        self.mean_arr_gpu = torch.zeros(n, dtype=torch.float32, device=self.device)
        self.align_bit_weights_gpu: Optional[torch.Tensor] = None
        self.tap_major_weights_gpu: Optional[torch.Tensor] = None    # xnor_b200_tap_major_weights copy, for channel-mask input
        self.output_gpu = torch.empty(batch, n, g.out_h, g.out_w, dtype=torch.float32, device=self.device)
        # zero-filled: when producers write this operand through sinks, padding taps and row tails are never written
        self.scratch = torch.zeros(capi.lib().xnor_b200_scratch_bytes(C.byref(self.desc)), dtype=torch.uint8, device=self.device)
        self.window_major = False      # operand rows in 2x2-window-major pixel order (set when a sink of this layer pools)
        self.bin_conv_shortcut_in_gpu: Optional[torch.Tensor] = None
        self.bin_conv_shortcut_out_gpu: Optional[torch.Tensor] = None
        self.shortcut_signs_gpu: Optional[torch.Tensor] = None       # sign words of the fused shortcut sum, when a layer reads them

    def load_weights(self, weights: torch.Tensor, biases: torch.Tensor) -> None:
        self.weights_gpu.copy_(weights.reshape(self.n, -1))
        self.biases_gpu.copy_(biases)


def make_convolutional_layer(batch, h, w, c, n, size, stride, pad, activation, xnor=1, device="cuda:0") -> ConvolutionalLayer:
    """make_convolutional_layer (src-lib/convolutional_layer.cpp:715), xnor layers only."""
    if not xnor:
        raise ValueError("this package implements the xnor=1 path only")
    return ConvolutionalLayer(batch, h, w, c, n, size, stride, pad, activation, device)


def binarize_weights(weights: torch.Tensor, n: int, size: int):
    """binarize_weights (src-lib/convolutional_layer.cpp:196): returns (binary [n][size], mean [n])."""
    binary = torch.empty(n, size, dtype=torch.float32, device=weights.device)
    mean = torch.empty(n, dtype=torch.float32, device=weights.device)
    capi.check(capi.lib().xnor_b200_binarize_weights(weights.data_ptr(), n, size, binary.data_ptr(), mean.data_ptr(), _stream()),
               "xnor_b200_binarize_weights")
    return binary, mean


def binary_align_weights(l: ConvolutionalLayer, invert: bool = False) -> None:
    """binary_align_weights (src-lib/convolutional_layer.cpp:1339): fills align_bit_weights_gpu and mean_arr_gpu."""
    l.align_bit_weights_gpu = torch.empty(l.geom.weights_bytes, dtype=torch.uint8, device=l.device)
    capi.check(capi.lib().xnor_b200_binary_align_weights(C.byref(l.desc), l.weights_gpu.data_ptr(),
                                                        l.align_bit_weights_gpu.data_ptr(), l.mean_arr_gpu.data_ptr(),
                                                        int(invert), _stream()), "xnor_b200_binary_align_weights")


def pack_input(l: ConvolutionalLayer, x: torch.Tensor) -> torch.Tensor:
    """The packed, transposed activation operand (t_bit_input) of every image: uint8 [batch*N][new_ldb/8]."""
    out = torch.empty(l.batch * l.geom.n_out, l.new_lda // 8, dtype=torch.uint8, device=l.device)
    capi.check(capi.lib().xnor_b200_pack_input(C.byref(l.desc), x.data_ptr(), out.data_ptr(), _stream()), "xnor_b200_pack_input")
    return out


def pack_input_staged(l: ConvolutionalLayer, x: torch.Tensor) -> torch.Tensor:
    """pack_input through the two-pass route (sign words first, rows from the words); c % 32 == 0 only."""
    out = torch.empty(l.batch * l.geom.n_out, l.new_lda // 8, dtype=torch.uint8, device=l.device)
    words = torch.empty(capi.lib().xnor_b200_pack_words_bytes(C.byref(l.desc)), dtype=torch.uint8, device=l.device)
    capi.check(capi.lib().xnor_b200_pack_input_staged(C.byref(l.desc), x.data_ptr(), words.data_ptr(), out.data_ptr(), _stream()),
               "xnor_b200_pack_input_staged")
    return out


def gemm_nn_custom_bin_mean_transposed_gpu(M, N, K, A, lda, B, ldb, C_out, ldc, mean_arr, bias, leaky,
                                           shortcut_in=None, shortcut_out=None) -> None:
    """gemm_nn_custom_bin_mean_transposed_gpu (src-lib/im2col_kernels.cu:1156), non-inverted A."""
    capi.check(capi.lib().xnor_b200_gemm_bin_mean_transposed(M, N, K, A.data_ptr(), lda, B.data_ptr(), ldb, C_out.data_ptr(), ldc,
                                                            mean_arr.data_ptr(), _ptr(bias), int(leaky), _ptr(shortcut_in),
                                                            _ptr(shortcut_out), _stream()), "xnor_b200_gemm_bin_mean_transposed")


def gemm_counts(M, N, K, A, lda, B, ldb) -> torch.Tensor:
    counts = torch.empty(M, N, dtype=torch.int32, device=A.device)
    capi.check(capi.lib().xnor_b200_gemm_counts(M, N, K, A.data_ptr(), lda, B.data_ptr(), ldb, counts.data_ptr(), _stream()),
               "xnor_b200_gemm_counts")
    return counts


def pack_input_pooled(l: ConvolutionalLayer, pool: capi.PoolDesc, x: torch.Tensor) -> torch.Tensor:
    """pack_input of maxpool(x) without materialising the pooled tensor; x is the maxpool's input."""
    out = torch.empty(l.batch * l.geom.n_out, l.new_lda // 8, dtype=torch.uint8, device=l.device)
    capi.check(capi.lib().xnor_b200_pack_input_pooled(C.byref(l.desc), C.byref(pool), x.data_ptr(), out.data_ptr(), _stream()),
               "xnor_b200_pack_input_pooled")
    return out


def forward_convolutional_layer_gpu(l: ConvolutionalLayer, x: torch.Tensor, pool: Optional[capi.PoolDesc] = None) -> torch.Tensor:
    """The xnor branch of forward_convolutional_layer_gpu (src-lib/convolutional_kernels.cu:204-262), whole batch.
    With `pool`, x is the input of a [maxpool] layer that sits directly in front of this convolution."""
    if l.align_bit_weights_gpu is None:
        raise RuntimeError("binary_align_weights() has not been called for this layer")
    expect = l.batch * l.c * (l.h * l.w if pool is None else pool.in_h * pool.in_w)
    if x.dtype != torch.float32 or not x.is_contiguous() or x.numel() != expect:
        raise ValueError("input must be a contiguous fp32 tensor of batch*c*h*w elements")
    if pool is not None:
        capi.check(capi.lib().xnor_b200_conv_forward_pooled(C.byref(l.desc), C.byref(pool), x.data_ptr(), l.align_bit_weights_gpu.data_ptr(),
                                                           l.mean_arr_gpu.data_ptr(), l.biases_gpu.data_ptr(), l.output_gpu.data_ptr(),
                                                           _ptr(l.bin_conv_shortcut_in_gpu), _ptr(l.bin_conv_shortcut_out_gpu),
                                                           l.scratch.data_ptr(), l.scratch.numel(), _stream()), "xnor_b200_conv_forward_pooled")
        return l.output_gpu
    capi.check(capi.lib().xnor_b200_conv_forward(C.byref(l.desc), x.data_ptr(), l.align_bit_weights_gpu.data_ptr(),
                                                l.mean_arr_gpu.data_ptr(), l.biases_gpu.data_ptr(), l.output_gpu.data_ptr(),
                                                _ptr(l.bin_conv_shortcut_in_gpu), _ptr(l.bin_conv_shortcut_out_gpu),
                                                l.scratch.data_ptr(), l.scratch.numel(), _stream()), "xnor_b200_conv_forward")
    return l.output_gpu


class Sink:
    """One direct consumer of a layer's sign bits (struct xnor_b200_sign_sink): `consumer` is the ConvolutionalLayer
    whose scratch the bits are written into, already in its packed-operand layout."""

    def __init__(self, consumer: "ConvolutionalLayer", channel_offset: int = 0, pool: int = 0, upsample: int = 0) -> None:
        self.consumer, self.channel_offset, self.pool, self.upsample = consumer, channel_offset, pool, upsample


def forward_convolutional_layer_io(l: ConvolutionalLayer, x: Optional[torch.Tensor] = None, x_signs: Optional[torch.Tensor] = None,
                                   pool: Optional[capi.PoolDesc] = None, want_signs: bool = False, packed: bool = False,
                                   sinks=(), want_output: Optional[bool] = None, x_masks: Optional[torch.Tensor] = None,
                                   shortcut_only: bool = False, shortcut_signs: bool = False,
                                   shortcut_sink: Optional["ConvolutionalLayer"] = None) -> Optional[torch.Tensor]:
    """xnor_b200_conv_forward_io.  Input: fp32 `x`, sign words / planes `x_signs`, or `packed` (the producers' sinks have
    filled l.scratch).  Output: the fp32 tensor (default when there are no sinks, or with want_output), the sign words
    int32 [batch][n/32][out_h*out_w] (want_signs), and/or the consumers' operands (sinks).  shortcut_only: only the fused
    shortcut sum (l.bin_conv_shortcut_out_gpu) is written and returned; the layer's own tensor is left untouched.
    shortcut_signs: the sign words of the sum are written to l.shortcut_signs_gpu as well.  shortcut_sink: the 1x1 layer
    that reads the sum; the signs go straight into its packed operand (its scratch)."""
    if l.align_bit_weights_gpu is None:
        raise RuntimeError("binary_align_weights() has not been called for this layer")
    io = capi.ConvIO()
    io.input = _ptr(x)
    io.input_signs = _ptr(x_signs)
    io.pool = C.pointer(pool) if pool is not None else None
    io.input_packed = int(packed)
    io.window_major = int(l.window_major)
    weights = l.align_bit_weights_gpu
    if x_masks is not None:
        if l.tap_major_weights_gpu is None:
            tap_major_weights(l)
        io.input_masks = x_masks.data_ptr()
        io.tap_major_weights = 1
        weights = l.tap_major_weights_gpu
    if want_output is None:
        want_output = not want_signs and not sinks
    out = None
    if want_signs:
        out = torch.empty(l.batch, l.n // 32, l.geom.n_out, dtype=torch.int32, device=l.device)
        io.output_signs = out.data_ptr()
    elif shortcut_only:
        out = l.bin_conv_shortcut_out_gpu
        io.shortcut_in = _ptr(l.bin_conv_shortcut_in_gpu)
        io.shortcut_out = out.data_ptr()
    elif want_output:
        out = l.output_gpu
        io.output = out.data_ptr()
        io.shortcut_in = _ptr(l.bin_conv_shortcut_in_gpu)
        io.shortcut_out = _ptr(l.bin_conv_shortcut_out_gpu)
    if shortcut_signs:
        if l.shortcut_signs_gpu is None:
            l.shortcut_signs_gpu = torch.empty(l.batch, l.n // 32, l.geom.n_out, dtype=torch.int32, device=l.device)
        io.shortcut_signs = l.shortcut_signs_gpu.data_ptr()
    if shortcut_sink is not None:
        sk = capi.SignSink()
        sk.consumer = C.pointer(shortcut_sink.desc)
        sk.consumer_scratch = shortcut_sink.scratch.data_ptr()
        sk.consumer_window_major = int(shortcut_sink.window_major)      # refused by the library: the epilogue writes row-major rows
        io.shortcut_sink = C.pointer(sk)
    if sinks:
        arr = (capi.SignSink * len(sinks))()
        for i, s in enumerate(sinks):
            arr[i].consumer = C.pointer(s.consumer.desc)
            arr[i].consumer_scratch = s.consumer.scratch.data_ptr()
            arr[i].channel_offset = s.channel_offset
            arr[i].pool = s.pool
            arr[i].upsample = s.upsample
            arr[i].consumer_window_major = int(s.consumer.window_major)
        io.sinks = arr
        io.n_sinks = len(sinks)
    capi.check(capi.lib().xnor_b200_conv_forward_io(C.byref(l.desc), C.byref(io), weights.data_ptr(),
                                                   l.mean_arr_gpu.data_ptr(), l.biases_gpu.data_ptr(), l.scratch.data_ptr(),
                                                   l.scratch.numel(), _stream()), "xnor_b200_conv_forward_io")
    return out


def tap_major_weights(l: ConvolutionalLayer) -> None:
    """Fills l.tap_major_weights_gpu (xnor_b200_tap_major_weights): the packed weights in tap-major K order."""
    l.tap_major_weights_gpu = torch.empty_like(l.align_bit_weights_gpu)
    capi.check(capi.lib().xnor_b200_tap_major_weights(C.byref(l.desc), l.align_bit_weights_gpu.data_ptr(),
                                                     l.tap_major_weights_gpu.data_ptr(), _stream()), "xnor_b200_tap_major_weights")


def conv_takes_masks(l: ConvolutionalLayer) -> bool:
    return bool(capi.lib().xnor_b200_conv_takes_masks(C.byref(l.desc)))
