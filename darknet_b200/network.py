"""Host-side network runner for Darknet xnor networks: cfg parser, .weights reader/writer, load-time
preparation and the forward loop.

It mirrors the reference's call sequence (names kept):

    net = parse_network_cfg(cfg_path, batch)         # src-lib/weights.cpp:47, src-lib/darknet_cfg.cpp:797-1068
    load_weights(net, weights_path)                  # src-lib/weights.cpp:421
    fuse_conv_batchnorm(net)                         # src-lib/darknet_network.cpp:1667
    calculate_binary_weights(net)                    # src-lib/darknet_network.cpp:1778
    out = network_predict_gpu(net, x)                # src-lib/network_kernels.cu:709 -> forward_network_gpu :30

Every [convolutional] xnor=1 layer runs through libxnor_b200.so (this package's product).  The layers
around the path -- the float convolutions, maxpool, route, upsample, shortcut, avgpool, softmax and
the yolo/region activations -- are not part of it; like Darknet, which hands them to cuDNN and its own
small kernels, this runner hands them to cuDNN/ATen through torch, in fp32 with TF32 disabled.
Only the section types and keys that occur in the three shipped xnor cfgs are understood.
"""
from __future__ import annotations

import math
import os
import struct
import zlib
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch
import torch.nn.functional as F

from . import capi
from . import layer as L


# ---- cfg -----------------------------------------------------------------------------------------

def read_cfg(text: str) -> List[Tuple[str, Dict[str, str]]]:
    """INI-like sections in file order; '#' and ';' start comments; keys are stripped of blanks."""
    sections: List[Tuple[str, Dict[str, str]]] = []
    for raw in text.splitlines():
        line = raw.strip()
        if not line or line[0] in "#;":
            continue
        if line.startswith("["):
            sections.append((line.strip("[] \t").lower(), {}))
        elif "=" in line and sections:
            k, v = line.split("=", 1)
            sections[-1][1][k.strip()] = v.strip()
    return sections


@dataclass
class Layer:
    type: str
    index: int
    c: int = 0
    h: int = 0
    w: int = 0
    out_c: int = 0
    out_h: int = 0
    out_w: int = 0
    opts: Dict[str, str] = field(default_factory=dict)
    # convolutional
    n: int = 0
    size: int = 1
    stride: int = 1
    pad: int = 0
    activation: str = "linear"
    batch_normalize: int = 0
    xnor: int = 0
    use_bin_output: int = 0
    weights: Optional[np.ndarray] = None
    biases: Optional[np.ndarray] = None
    scales: Optional[np.ndarray] = None
    rolling_mean: Optional[np.ndarray] = None
    rolling_variance: Optional[np.ndarray] = None
    weights_gpu: Optional[torch.Tensor] = None
    biases_gpu: Optional[torch.Tensor] = None
    xnor_layer: Optional[L.ConvolutionalLayer] = None
    # route / shortcut
    input_layers: List[int] = field(default_factory=list)
    # shortcut fused into the preceding xnor conv (src-lib/darknet_network.cpp:1799-1813)
    blank: bool = False
    # maxpool whose only reader is the xnor conv right after it: folded into that conv's pack kernel
    folded: bool = False
    pool_desc: Optional[capi.PoolDesc] = None
    # xnor conv whose only reader is another xnor conv (directly or through a maxpool): hands over sign bits
    weights_blocked_gpu: Optional[torch.Tensor] = None     # float conv on a small map: weights re-blocked at load time
    branch_start: bool = False       # first / last layer of a head branch that runs on the side stream
    branch_end: bool = False
    yolo_entries: int = 0            # float conv in front of a [yolo] layer: the head's logistic step runs in the conv epilogue
    yolo_done: bool = False          # [yolo] layer whose activation the previous layer already applied
    conv3_pool: int = 0              # first float conv (3 channels, 3x3): 2 = the 2x2/2 maxpool behind it is applied in the kernel
    emit_planes: bool = False        # ... and only the sign planes of the pooled output are written
    emit_masks: bool = False         # ... as channel masks per pixel instead (the next layer's short-row GEMM reads them directly)
    mask_source: Optional[int] = None
    emit_signs: bool = False
    # direct sign sinks (xnor_b200_sign_sink): this xnor conv's epilogue fills the packed operand of later xnor convs
    sinks: List = field(default_factory=list)      # of L.Sink
    packed_input: bool = False       # xnor conv: every input channel arrives through producers' sinks
    need_fp32: bool = True           # somebody still reads this layer's fp32 output
    shortcut_only: bool = False      # xnor conv whose output only the fused [shortcut] behind it reads: just the sum is written
    emit_sum_signs: bool = False     # xnor conv with a fused [shortcut] whose sum the next xnor layer reads: also writes its sign words
    sum_sink_to: Optional[int] = None  # ... or, when that reader is a 1x1 layer, writes them into its packed operand (layer index)
    skip: bool = False               # maxpool / upsample / route that only sat between a sink producer and its consumer
    sign_source: Optional[int] = None
    sign_out: Optional[torch.Tensor] = None
    output_gpu: Optional[torch.Tensor] = None

    @property
    def outputs(self) -> int:
        return self.out_c * self.out_h * self.out_w


@dataclass
class Network:
    batch: int
    c: int
    h: int
    w: int
    layers: List[Layer]
    device: torch.device
    xnor_launches_per_forward: int = 0
    folded_maxpools: int = 0
    fold_maxpool_min_batch: int = 4
    sign_chains: bool = True
    skip_fused_conv_outputs: bool = True   # an xnor conv read only by its fused [shortcut] does not write its own tensor
    sum_signs_min_batch: int = 4           # from this batch on the sign of a fused shortcut sum is handed to the next xnor layer (the call runs on the tensor-core kernel; measured on darknet53: +5 % at batch 4, -7 % at batch 2, -26 % at batch 1)
    sum_sign_links: int = 0
    fuse_first_conv: bool = True
    float_map_max_pixels: int = 1024       # batch*out_h*out_w up to which float convs use the cluster split-K kernel (measured: it wins at 676 pixels, loses to cuDNN/cuBLAS at 1352)
    sign_links: int = 0
    heads_direct_to_host: bool = True      # with heads_host: a fused head convolution stores into the pinned host tensor itself
    side_branches: bool = True             # a head branch that nothing later reads runs on a second stream
    side_stream: Optional[torch.cuda.Stream] = None
    packed_from_cache: int = 0             # xnor layers whose packed weights came from the cache file beside the .weights file
    sink_max_batch: int = 1 << 30          # batch up to which direct sign sinks are linked (measured: a gain at every batch for yolov3-tiny, within 2% either way for the other two networks at batch 32-256)
    sink_links: int = 0


def parse_network_cfg(path: str, batch: int = 1, device: str = "cuda:0") -> Network:
    with open(path) as fh:
        sections = read_cfg(fh.read())
    if not sections or sections[0][0] not in ("net", "network"):
        raise ValueError("first cfg section must be [net]")
    net_opts = sections[0][1]
    c, h, w = int(net_opts.get("channels", 3)), int(net_opts.get("height", 0)), int(net_opts.get("width", 0))
    net = Network(batch, c, h, w, [], torch.device(device))
    for idx, (name, o) in enumerate(sections[1:]):
        l = Layer(name, idx, c, h, w, opts=o)
        if name == "convolutional":
            l.n = int(o.get("filters", 1))
            l.size = int(o.get("size", 1))
            l.stride = int(o.get("stride", 1))
            l.pad = l.size // 2 if int(o.get("pad", 0)) else int(o.get("padding", 0))
            l.activation = o.get("activation", "logistic")
            l.batch_normalize = int(o.get("batch_normalize", 0))
            l.xnor = int(o.get("xnor", 0))
            l.use_bin_output = int(o.get("bin_output", 0))
            l.out_c = l.n
            l.out_h = (h + 2 * l.pad - l.size) // l.stride + 1
            l.out_w = (w + 2 * l.pad - l.size) // l.stride + 1
        elif name == "maxpool":
            l.stride = int(o.get("stride", 1))                    # defaults as in src-lib/darknet_cfg.cpp:1597-1601
            l.size = int(o.get("size", l.stride))
            l.pad = int(o.get("padding", l.size - 1))
            l.out_c = c
            l.out_h = (h + l.pad - l.size) // l.stride + 1       # src-lib/maxpool_layer.cpp:129-130
            l.out_w = (w + l.pad - l.size) // l.stride + 1
        elif name == "route":
            refs = [int(v) for v in o["layers"].split(",")]
            l.input_layers = [r if r >= 0 else idx + r for r in refs]
            first = net.layers[l.input_layers[0]]
            l.out_h, l.out_w = first.out_h, first.out_w
            l.out_c = sum(net.layers[i].out_c for i in l.input_layers)
            for i in l.input_layers:                              # src-lib/darknet_cfg.cpp:833-845
                net.layers[i].use_bin_output = 0
        elif name == "shortcut":
            frm = int(o["from"])
            l.input_layers = [frm if frm >= 0 else idx + frm]
            l.activation = o.get("activation", "linear")
            l.out_c, l.out_h, l.out_w = c, h, w
            net.layers[idx - 1].use_bin_output = 0               # src-lib/darknet_cfg.cpp:846-856
            net.layers[l.input_layers[0]].use_bin_output = 0
        elif name == "upsample":
            l.stride = int(o.get("stride", 2))
            l.out_c, l.out_h, l.out_w = c, h * l.stride, w * l.stride
        elif name == "avgpool":
            l.out_c, l.out_h, l.out_w = c, 1, 1
        elif name in ("yolo", "region", "softmax"):
            l.out_c, l.out_h, l.out_w = c, h, w
        else:
            raise ValueError(f"cfg section [{name}] is outside the xnor cfgs this runner understands")
        net.layers.append(l)
        c, h, w = l.out_c, l.out_h, l.out_w
    return net


# ---- .weights ------------------------------------------------------------------------------------
# header: int32 major, minor, revision; `seen` uint64 when major*10+minor >= 2 else uint32
# (src-lib/weights.cpp:460-478); per conv: biases[n], then scales/rolling_mean/rolling_variance[n] when
# batch_normalize, then weights[n*c*size*size] fp32 (src-lib/weights.cpp:369-398).

def write_synthetic_weights(net: Network, path: str, seed: int = 1, random_batchnorm: bool = False, exact_first_conv: bool = False) -> None:
    """Seeded weights: w ~ N(0, 0.05), b ~ N(0, 0.01), BN scales 1, rolling mean 0, rolling variance 1.
    random_batchnorm: scales, means and variances drawn at random instead (exercises fuse_conv_batchnorm).
    exact_first_conv: the first convolution's weights and biases are multiples of 2^-10 and its rolling variance makes the
    batch-norm factor round to one, so that with inputs on a 2^-8 grid every partial sum of that layer is exact in fp32 and
    two implementations that add in different orders still produce bit-identical activations."""
    rng = np.random.default_rng(seed)
    first = True
    with open(path, "wb") as fh:
        fh.write(struct.pack("<iiiQ", 0, 2, 5, 0))
        for l in net.layers:
            if l.type != "convolutional":
                continue
            exact = exact_first_conv and first
            first = False
            b = rng.standard_normal(l.n) * 0.01
            w = rng.standard_normal(l.n * l.c * l.size * l.size) * 0.05
            if exact:
                b, w = np.round(b * 1024) / 1024, np.clip(np.round(w * 1024) / 1024, -0.25, 0.25)
            fh.write(b.astype("<f4").tobytes())
            if l.batch_normalize:
                if random_batchnorm and not exact:
                    fh.write((0.5 + rng.random(l.n)).astype("<f4").tobytes())
                    fh.write((rng.standard_normal(l.n) * 0.1).astype("<f4").tobytes())
                    fh.write((0.25 + rng.random(l.n)).astype("<f4").tobytes())
                else:
                    fh.write(np.ones(l.n, "<f4").tobytes())
                    fh.write(np.zeros(l.n, "<f4").tobytes())
                    # 1 - 1e-5: sqrt(variance + 1e-5) is then within 1e-8 of one and weights on a coarse grid stay as they are
                    fh.write(np.full(l.n, 1.0 - 1e-5 if exact else 1.0, "<f4").tobytes())
            fh.write(w.astype("<f4").tobytes())


def load_weights(net: Network, path: str) -> None:
    with open(path, "rb") as fh:
        major, minor, _rev = struct.unpack("<iii", fh.read(12))
        fh.read(8 if major * 10 + minor >= 2 else 4)

        def take(count: int) -> np.ndarray:
            buf = fh.read(4 * count)
            if len(buf) != 4 * count:
                raise ValueError("weights file ended early")
            return np.frombuffer(buf, "<f4").astype(np.float32)

        for l in net.layers:
            if l.type != "convolutional":
                continue
            l.biases = take(l.n)
            if l.batch_normalize:
                l.scales, l.rolling_mean, l.rolling_variance = take(l.n), take(l.n), take(l.n)
            l.weights = take(l.n * l.c * l.size * l.size).reshape(l.n, l.c, l.size, l.size)


# ---- packed-weight cache -------------------------------------------------------------------------
# Darknet carries a dormant writer for bit-packed weights (save_convolutional_weights_binary, src-lib/weights.cpp:70-116:
# per filter the mean and size/8 bytes of sign bits) and re-packs every xnor layer in a host triple loop at each load
# (src-lib/convolutional_layer.cpp:1371-1391).  The cache keeps what the path actually consumes -- align_bit_weights in its
# final K order with the row padding, and mean_arr -- beside the .weights file, keyed by the layer geometry and a CRC of
# the batch-norm-folded fp32 weights it was packed from, so a stale or foreign file is never used.
#
# file: "XNORPACK" | u32 version | u32 entries | entries | u32 crc32 of everything before it
# entry: i32 layer index, c, n, size, stride, pad, new_lda | u32 crc32(fp32 weights) | u64 bits bytes | bits | f32 mean[n]

PACK_MAGIC = b"XNORPACK"
PACK_VERSION = 1


def packed_cache_path(weights_path: str) -> str:
    return weights_path + ".xnorpack"


def weights_crc(l: Layer) -> int:
    """CRC-32 of the layer's fp32 weights as the packer sees them (after fuse_conv_batchnorm)."""
    return zlib.crc32(np.ascontiguousarray(l.weights, "<f4").tobytes()) & 0xFFFFFFFF


def write_packed_cache(path: str, entries: List[dict]) -> None:
    """entries: dicts with index, c, n, size, stride, pad, new_lda, crc, bits (uint8 [n*new_lda/8]), mean (float32 [n])."""
    body = bytearray(PACK_MAGIC + struct.pack("<II", PACK_VERSION, len(entries)))
    for e in entries:
        bits = np.ascontiguousarray(e["bits"], np.uint8)
        mean = np.ascontiguousarray(e["mean"], "<f4")
        if bits.size != e["n"] * e["new_lda"] // 8 or mean.size != e["n"]:
            raise ValueError("packed-weight entry has the wrong size")
        body += struct.pack("<7iIQ", e["index"], e["c"], e["n"], e["size"], e["stride"], e["pad"], e["new_lda"], e["crc"], bits.size)
        body += bits.tobytes() + mean.tobytes()
    body += struct.pack("<I", zlib.crc32(bytes(body)) & 0xFFFFFFFF)
    tmp = path + ".tmp"
    with open(tmp, "wb") as fh:
        fh.write(body)
    os.replace(tmp, path)


def read_packed_cache(path: str) -> Dict[int, dict]:
    """Layer index -> entry.  Raises ValueError on a damaged, truncated or foreign file."""
    with open(path, "rb") as fh:
        data = fh.read()
    if len(data) < 20 or data[:8] != PACK_MAGIC:
        raise ValueError("not a packed-weight cache")
    if zlib.crc32(data[:-4]) & 0xFFFFFFFF != struct.unpack("<I", data[-4:])[0]:
        raise ValueError("packed-weight cache is damaged (checksum)")
    version, count = struct.unpack_from("<II", data, 8)
    if version != PACK_VERSION:
        raise ValueError("packed-weight cache has another version")
    out: Dict[int, dict] = {}
    off = 16
    for _ in range(count):
        index, c, n, size, stride, pad, new_lda, crc, nbytes = struct.unpack_from("<7iIQ", data, off)
        off += struct.calcsize("<7iIQ")
        if n <= 0 or new_lda <= 0 or nbytes != n * new_lda // 8 or off + nbytes + 4 * n > len(data) - 4:
            raise ValueError("packed-weight cache entry is inconsistent")
        bits = np.frombuffer(data, np.uint8, nbytes, off).copy()
        off += nbytes
        mean = np.frombuffer(data, "<f4", n, off).astype(np.float32)
        off += 4 * n
        out[index] = dict(index=index, c=c, n=n, size=size, stride=stride, pad=pad, new_lda=new_lda, crc=crc, bits=bits, mean=mean)
    return out


def cache_entry_matches(e: Optional[dict], l: Layer, new_lda: int) -> bool:
    return (e is not None and (e["c"], e["n"], e["size"], e["stride"], e["pad"], e["new_lda"]) == (l.c, l.n, l.size, l.stride, l.pad, new_lda)
            and e["crc"] == weights_crc(l))


def packed_entries(net: Network) -> List[dict]:
    """What the loaded network holds, ready for write_packed_cache."""
    out = []
    for l in net.layers:
        if l.type == "convolutional" and l.xnor and l.xnor_layer is not None:
            xl = l.xnor_layer
            out.append(dict(index=l.index, c=l.c, n=l.n, size=l.size, stride=l.stride, pad=l.pad, new_lda=xl.new_lda, crc=weights_crc(l),
                            bits=xl.align_bit_weights_gpu.cpu().numpy(), mean=xl.mean_arr_gpu.cpu().numpy()))
    return out


# ---- load-time preparation -----------------------------------------------------------------------

def fuse_conv_batchnorm(net: Network) -> None:
    """Folds batch-norm into weights and biases in double precision (src-lib/darknet_network.cpp:1667-1708)."""
    for l in net.layers:
        if l.type == "convolutional" and l.batch_normalize:
            std = np.sqrt(l.rolling_variance.astype(np.float64) + 0.00001)
            l.biases = (l.biases.astype(np.float64) - l.scales.astype(np.float64) * l.rolling_mean.astype(np.float64) / std).astype(np.float32)
            pre = l.scales.astype(np.float64) / std
            l.weights = (l.weights.astype(np.float64) * pre[:, None, None, None]).astype(np.float32)
            l.batch_normalize = 0


def calculate_binary_weights(net: Network, packed: Optional[Dict[int, dict]] = None) -> None:
    """Packs every xnor conv through the C ABI (or takes its packed weights from `packed`, the entries of a cache file,
    where geometry and weight checksum match), drops the activation of bin_output layers and fuses a same-shape
    [shortcut] that directly follows an xnor conv (src-lib/darknet_network.cpp:1778-1817)."""
    dev = net.device
    for j, l in enumerate(net.layers):
        if l.type != "convolutional":
            continue
        l.weights_gpu = torch.from_numpy(l.weights).to(dev)
        l.biases_gpu = torch.from_numpy(l.biases).to(dev)
        if not l.xnor:
            continue
        if l.use_bin_output:
            l.activation = "linear"
        if l.activation not in ("linear", "leaky"):
            raise ValueError("xnor layers in the shipped cfgs are leaky or linear")
        act = capi.LEAKY if l.activation == "leaky" else capi.LINEAR
        xl = L.make_convolutional_layer(net.batch, l.h, l.w, l.c, l.n, l.size, l.stride, l.pad, act, device=str(dev))
        xl.load_weights(l.weights_gpu, l.biases_gpu)
        cached = packed.get(j) if packed else None
        if cache_entry_matches(cached, l, xl.new_lda):
            xl.align_bit_weights_gpu = torch.from_numpy(cached["bits"]).to(dev)
            xl.mean_arr_gpu.copy_(torch.from_numpy(cached["mean"]))
            net.packed_from_cache += 1
        else:
            L.binary_align_weights(xl)
        l.xnor_layer = xl
        l.output_gpu = xl.output_gpu
        net.xnor_launches_per_forward += 2
        if j + 1 < len(net.layers):
            sc = net.layers[j + 1]
            # Darknet's GPU build fuses whatever the [shortcut]'s activation is and thereby drops it (the blanked layer does
            # nothing); its CPU build applies it.  Only a linear shortcut is fused here, so both semantics coincide.
            if sc.type == "shortcut" and (sc.w, sc.h, sc.c) == (sc.out_w, sc.out_h, sc.out_c) and sc.activation == "linear":
                sc.blank = True
                sc.output_gpu = torch.empty(net.batch, sc.out_c, sc.out_h, sc.out_w, device=dev)
                xl.bin_conv_shortcut_out_gpu = sc.output_gpu
    readers = _readers(net)
    for j, l in enumerate(net.layers[:-1]):
        # Darknet's fused kernel writes the convolution's own tensor and the sum (src-lib/im2col_kernels.cu:940-953); with the
        # [shortcut] layer blanked nothing reads the former, and at large batch it is a third of the layer's memory traffic
        l.shortcut_only = (net.skip_fused_conv_outputs and l.type == "convolutional" and l.xnor and net.layers[j + 1].blank
                           and readers[j] == [j + 1])
    prepare_float_map_convs(net)
    link_branches(net)
    if net.sign_chains:
        link_sinks(net)
        link_sign_chains(net)
        link_shortcut_sums(net)
        for l in net.layers:
            if l.emit_sum_signs:
                l.xnor_layer.shortcut_signs_gpu = torch.empty(net.batch, l.n // 32, l.out_h * l.out_w, dtype=torch.int32, device=dev)
    if net.fuse_first_conv:
        link_first_conv(net)
    fold_maxpools(net)
    torch.cuda.synchronize(dev)


def _readers(net: Network) -> Dict[int, List[int]]:
    """Layer index -> indices of the layers that read its output."""
    out: Dict[int, List[int]] = {i: [] for i in range(len(net.layers))}
    for k, l in enumerate(net.layers):
        if l.type == "route":
            for i in l.input_layers:
                out[i].append(k)
            continue
        if k > 0:
            out[k - 1].append(k)
        if l.type == "shortcut":
            for i in l.input_layers:
                out[i].append(k)
    return out


def link_branches(net: Network) -> None:
    """A [route] with one input i < k-1 starts a second branch at layer i; when nothing at or behind the route reads the
    layers i+1 .. k-1 (they end in a detection head), those layers are independent of everything that follows and run
    on a side stream, concurrently with the rest of the network.  Every kernel of a batch-1 forward fills a fraction of
    the GPU, so the two branches overlap almost completely."""
    if not net.side_branches:
        return
    readers = _readers(net)
    for k, r in enumerate(net.layers):
        if r.type != "route" or len(r.input_layers) != 1 or r.input_layers[0] >= k - 1:
            continue
        i = r.input_layers[0]
        inside = set(range(i + 1, k))
        if all(set(readers[j]) <= inside for j in inside) and not any(net.layers[j].branch_start for j in inside):
            net.layers[i + 1].branch_start = True
            net.layers[k - 1].branch_end = True


def link_sinks(net: Network) -> None:
    """Finds xnor convolutions whose whole input comes from other xnor convolutions through nothing but a 2x2/stride-2
    [maxpool], a stride-2 [upsample] or a [route]: those producers then write the consumer's packed operand from their
    GEMM epilogue (sign sinks), the consumer runs without a pack kernel, and the layers in between are skipped when
    nobody else reads them.  A producer keeps its fp32 output only if some other layer reads it."""
    if net.batch > net.sink_max_batch:
        return
    layers = net.layers
    readers = _readers(net)

    def resolve(k: int, pool: int, up: int):
        """Input expression of a consumer, walked backwards from layer k: [(producer, channel offset, pool, up, via)]."""
        l = layers[k]
        if l.type == "convolutional":
            if l.xnor and l.xnor_layer is not None and l.n % 32 == 0 and not (k + 1 < len(layers) and layers[k + 1].blank):
                return [(k, 0, pool, up, [])]
            return None
        if l.type == "maxpool" and pool == 0 and up == 0 and k > 0:
            if l.size == 2 and l.stride == 2 and l.pad // 2 == 0 and l.h % 2 == 0 and l.w % 2 == 0 and not l.folded:
                r = resolve(k - 1, 2, 0)
                return None if r is None else [(p, o, pl, u, via + [k]) for p, o, pl, u, via in r]
            return None
        if l.type == "upsample" and pool == 0 and up == 0 and l.stride == 2 and k > 0:
            r = resolve(k - 1, 0, 2)
            return None if r is None else [(p, o, pl, u, via + [k]) for p, o, pl, u, via in r]
        if l.type == "route":
            parts, off = [], 0
            for i in l.input_layers:
                r = resolve(i, pool, up)
                if r is None or off % 32 != 0:
                    return None
                parts += [(p, o + off, pl, u, via + [k]) for p, o, pl, u, via in r]
                off += layers[i].out_c
            return parts
        return None

    for k, c in enumerate(layers):
        if not (c.type == "convolutional" and c.xnor and c.xnor_layer is not None and c.c % 32 == 0 and c.stride == 1
                and 2 * c.pad == c.size - 1 and k > 0 and c.pool_desc is None and c.sign_source is None):
            continue
        expr = resolve(k - 1, 0, 0)
        if expr is None:
            continue
        if any(len(layers[p].sinks) >= 2 for p, *_ in expr):
            continue
        c.packed_input = True
        for p, off, pool, up, via in expr:
            layers[p].sinks.append(L.Sink(c.xnor_layer, off, pool, up))
            if pool == 2:
                layers[p].xnor_layer.window_major = True
            net.sink_links += 1
    # which fp32 tensors are still read: walk backwards, a packed consumer reads none
    for k in range(len(layers) - 1, -1, -1):
        l = layers[k]
        if not readers[k]:
            l.need_fp32 = True                       # network output
            continue
        need = False
        for r in readers[k]:
            rl = layers[r]
            if rl.type == "convolutional" and rl.packed_input:
                continue
            if rl.type in ("maxpool", "upsample", "route") and not rl.need_fp32:
                continue
            need = True
        l.need_fp32 = need
        if l.type in ("maxpool", "upsample", "route") and not need:
            l.skip = True


def link_shortcut_sums(net: Network) -> None:
    """conv j + fused [shortcut] j+1 -> xnor conv j+2: the consumer takes the sign of the sum instead of the fp32 sum, as
    channel-packed words that its pack kernel reads (emit_sum_signs), or -- a 1x1 reader over exactly these filters --
    straight into its packed operand (sum_sink_to; it then runs without a pack kernel).  Runs after link_sinks: the
    epilogue writes that operand in row-major pixel order, so a reader that link_sinks made window-major (it feeds a
    pooled sink of its own) takes the words instead."""
    if net.batch < net.sum_signs_min_batch:
        return
    for j, l in enumerate(net.layers[:-2]):
        nxt = net.layers[j + 2]
        if not (l.type == "convolutional" and l.xnor and net.layers[j + 1].blank and l.n % 32 == 0
                and nxt.type == "convolutional" and nxt.xnor and nxt.xnor_layer is not None and nxt.c % 32 == 0):
            continue
        if nxt.packed_input or nxt.sign_source is not None or nxt.pool_desc is not None:
            continue
        if nxt.size == 1 and nxt.stride == 1 and nxt.pad == 0 and nxt.c == l.n and not nxt.xnor_layer.window_major:
            l.sum_sink_to = j + 2
            nxt.packed_input = True
        else:
            l.emit_sum_signs = True
            nxt.sign_source = j + 1
        net.sum_sign_links += 1


def link_sign_chains(net: Network) -> None:
    """Finds xnor convolutions whose output is read by nothing but the next xnor convolution -- directly or through
    one [maxpool] -- and switches the pair to the sign-bit hand-over of xnor_b200_conv_forward_io: the producer
    writes 1 bit per value, the maxpool becomes an OR inside the consumer's pack kernel, and neither the fp32
    tensor nor the pooled tensor exists.  These are the bin_output=1 layers of the tiny networks."""
    referenced = set()
    for l in net.layers:
        if l.type in ("route", "shortcut"):
            referenced.update(l.input_layers)
    n = len(net.layers)
    for j, l in enumerate(net.layers):
        if not (l.type == "convolutional" and l.xnor and l.xnor_layer is not None and l.n % 32 == 0) or j in referenced or j + 1 >= n:
            continue
        if l.sinks:
            continue
        if net.layers[j + 1].blank:
            continue
        k = j + 1
        pool = None
        if net.layers[k].type == "maxpool" and k not in referenced and k + 1 < n:
            pool = net.layers[k]
            k += 1
        consumer = net.layers[k]
        if not (consumer.type == "convolutional" and consumer.xnor and consumer.xnor_layer is not None) or consumer.packed_input:
            continue
        l.emit_signs = True
        consumer.sign_source = j
        if pool is not None:
            pool.folded = True
            consumer.pool_desc = capi.PoolDesc(pool.size, pool.stride, pool.pad, pool.h, pool.w)
        net.sign_links += 1


def link_first_conv(net: Network) -> None:
    """The float 3-channel 3x3 convolution in front of the path: when a 2x2/stride-2 [maxpool] that nothing else reads
    follows it, the kernel pools in registers; when the layer after that is an xnor convolution (c % 32 != 0, so it
    takes x-packed sign planes) the kernel writes just those planes (xnor_b200_float_conv3_io)."""
    referenced = set()
    for l in net.layers:
        if l.type in ("route", "shortcut"):
            referenced.update(l.input_layers)
    for j, l in enumerate(net.layers):
        if not (l.type == "convolutional" and not l.xnor and l.c == 3 and l.size == 3 and l.stride == 1 and l.pad == 1
                and l.activation in ("leaky", "linear")):
            continue
        if j in referenced or j + 1 >= len(net.layers):
            continue
        nxt = net.layers[j + 1]
        if (net.sign_chains and l.n == 32 and nxt.type == "convolutional" and nxt.xnor and nxt.xnor_layer is not None and nxt.c == 32
                and nxt.pool_desc is None):
            # 32 filters straight into an xnor layer: the kernel writes one sign word per pixel, no fp32 tensor
            l.emit_masks = True
            nxt.sign_source = j
            net.sign_links += 1
            continue
        mp = net.layers[j + 1]
        if not (mp.type == "maxpool" and not mp.folded and mp.size == 2 and mp.stride == 2 and mp.pad // 2 == 0
                and mp.h % 2 == 0 and mp.w % 2 == 0):
            continue
        l.conv3_pool = 2
        mp.folded = True
        if net.sign_chains and j + 1 not in referenced and j + 2 < len(net.layers):
            nxt = net.layers[j + 2]
            if nxt.type == "convolutional" and nxt.xnor and nxt.xnor_layer is not None and nxt.c % 32 != 0 and nxt.pool_desc is None:
                if L.conv_takes_masks(nxt.xnor_layer):
                    l.emit_masks = True
                    nxt.mask_source = j
                    L.tap_major_weights(nxt.xnor_layer)
                else:
                    l.emit_planes = True
                    nxt.sign_source = j
                net.sign_links += 1


def fold_maxpools(net: Network) -> None:
    """Marks every [maxpool] that only feeds the xnor convolution directly after it: the convolution then reads the
    maxpool's input and pools while packing (xnor_b200_conv_forward_pooled), and the maxpool layer does nothing."""
    referenced = set()
    for l in net.layers:
        if l.type in ("route", "shortcut"):
            referenced.update(l.input_layers)
    for j, l in enumerate(net.layers[:-1]):
        nxt = net.layers[j + 1]
        # Measured on B200: the folded kernel wins from a few images per call upwards (it reads the unpooled tensor
        # once instead of writing and re-reading the pooled one) and only for the 2x2/stride-2 window it has a
        # vectorised path for; at batch 1 the separate maxpool launch is cheaper than the longer pack kernel.
        fast = l.size == 2 and l.stride == 2 and l.pad // 2 == 0 and l.h % 2 == 0 and l.w % 2 == 0
        if (l.type == "maxpool" and not l.folded and not l.skip and j not in referenced and nxt.type == "convolutional" and nxt.xnor and nxt.xnor_layer is not None
                and fast and net.batch >= net.fold_maxpool_min_batch):
            l.folded = True
            nxt.pool_desc = capi.PoolDesc(l.size, l.stride, l.pad, l.h, l.w)
            net.folded_maxpools += 1


# ---- forward -------------------------------------------------------------------------------------

def _activate(x: torch.Tensor, a: str) -> torch.Tensor:
    if a == "linear":
        return x
    if a == "leaky":
        return F.leaky_relu(x, 0.1)
    if a == "logistic":
        return torch.sigmoid(x)
    raise ValueError(f"activation {a} not used by the xnor cfgs")


def _float_conv3(net: Network, l: Layer, x: torch.Tensor) -> torch.Tensor:
    """The 3-channel 3x3 first convolution: 2x2 blocks per thread, optional fused maxpool, optional sign-plane output."""
    import ctypes as C
    desc = capi.ConvDesc(net.batch, l.c, l.h, l.w, l.n, l.size, l.stride, l.pad, capi.LEAKY if l.activation == "leaky" else capi.LINEAR)
    oh, ow = (l.out_h // 2, l.out_w // 2) if l.conv3_pool else (l.out_h, l.out_w)
    if l.emit_masks:
        out = torch.empty(net.batch, oh, ow, (l.n + 7) // 8, dtype=torch.uint8, device=x.device)
    elif l.emit_planes:
        out = torch.empty(net.batch, l.n, oh, (ow + 31) // 32, dtype=torch.int32, device=x.device)
    else:
        out = torch.empty(net.batch, l.n, oh, ow, dtype=torch.float32, device=x.device)
    fp32 = not (l.emit_planes or l.emit_masks)
    capi.check(capi.lib().xnor_b200_float_conv3_io(C.byref(desc), l.conv3_pool, x.data_ptr(), l.weights_gpu.data_ptr(), l.biases_gpu.data_ptr(),
                                                  out.data_ptr() if fp32 else None, out.data_ptr() if l.emit_planes else None,
                                                  out.data_ptr() if l.emit_masks else None,
                                                  torch.cuda.current_stream().cuda_stream), "xnor_b200_float_conv3_io")
    return out


def _float_conv_small(net: Network, l: Layer, x: torch.Tensor) -> torch.Tensor:
    """The few-input-channel float convolution in front of the path: one fused direct-convolution kernel."""
    import ctypes as C
    desc = capi.ConvDesc(net.batch, l.c, l.h, l.w, l.n, l.size, l.stride, l.pad, capi.LEAKY if l.activation == "leaky" else capi.LINEAR)
    out = torch.empty(net.batch, l.n, l.out_h, l.out_w, dtype=torch.float32, device=x.device)
    capi.check(capi.lib().xnor_b200_float_conv_small(C.byref(desc), x.data_ptr(), l.weights_gpu.data_ptr(), l.biases_gpu.data_ptr(),
                                                    out.data_ptr(), torch.cuda.current_stream().cuda_stream), "xnor_b200_float_conv_small")
    return out


def _map_conv_desc(net: Network, l: Layer) -> capi.ConvDesc:
    return capi.ConvDesc(net.batch, l.c, l.h, l.w, l.n, l.size, l.stride, l.pad, capi.LEAKY if l.activation == "leaky" else capi.LINEAR)


def prepare_float_map_convs(net: Network) -> None:
    """Re-blocks the weights of the float convolutions that the small-map kernel takes (many channels, stride 1,
    3x3/pad 1 or 1x1, few output pixels in the whole batch).  Runs after fuse_conv_batchnorm."""
    import ctypes as C
    for l in net.layers:
        if l.type != "convolutional" or l.xnor or l.activation not in ("leaky", "linear"):
            continue
        if l.c * l.size * l.size <= 128 or net.batch * l.out_h * l.out_w > net.float_map_max_pixels:
            continue
        desc = _map_conv_desc(net, l)
        nbytes = capi.lib().xnor_b200_float_conv_map_weights_bytes(C.byref(desc))
        if nbytes == 0:
            continue
        nxt = net.layers[l.index + 1] if l.index + 1 < len(net.layers) else None
        if (nxt is not None and nxt.type == "yolo" and l.activation == "linear" and float(nxt.opts.get("scale_x_y", 1)) == 1.0
                and l.n % (5 + int(nxt.opts.get("classes", 20))) == 0):
            l.yolo_entries = 5 + int(nxt.opts.get("classes", 20))
            nxt.yolo_done = True
        l.weights_blocked_gpu = torch.empty(nbytes // 4, dtype=torch.float32, device=l.weights_gpu.device)
        capi.check(capi.lib().xnor_b200_float_conv_map_prepare(C.byref(desc), l.weights_gpu.data_ptr(), l.weights_blocked_gpu.data_ptr(),
                                                              torch.cuda.current_stream().cuda_stream), "xnor_b200_float_conv_map_prepare")


def _float_conv_1x1_tc(l: Layer, x: torch.Tensor) -> torch.Tensor:
    """1x1 / stride-1 float convolution + bias + leaky/linear through xnor_b200_float_conv_1x1_tc."""
    import ctypes as C
    desc = capi.ConvDesc(x.shape[0], l.c, l.h, l.w, l.n, 1, 1, 0, capi.LEAKY if l.activation == "leaky" else capi.LINEAR)
    out = torch.empty(x.shape[0], l.n, l.out_h, l.out_w, dtype=torch.float32, device=x.device)
    capi.check(capi.lib().xnor_b200_float_conv_1x1_tc(C.byref(desc), x.data_ptr(), l.weights_gpu.data_ptr(), l.biases_gpu.data_ptr(),
                                                     out.data_ptr(), torch.cuda.current_stream().cuda_stream), "xnor_b200_float_conv_1x1_tc")
    return out


def _float_conv_map(net: Network, l: Layer, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """A many-channel float convolution on a small map: cluster split-K kernel with bias and activation fused.  `out` may be
    a pinned host tensor (the device writes a finished head straight into host memory)."""
    import ctypes as C
    desc = _map_conv_desc(net, l)
    if out is None:
        out = torch.empty(net.batch, l.n, l.out_h, l.out_w, dtype=torch.float32, device=x.device)
    capi.check(capi.lib().xnor_b200_float_conv_map_yolo(C.byref(desc), x.data_ptr(), l.weights_blocked_gpu.data_ptr(), l.biases_gpu.data_ptr(),
                                                       out.data_ptr(), l.yolo_entries, torch.cuda.current_stream().cuda_stream),
               "xnor_b200_float_conv_map_yolo")
    return out


def _maxpool(x: torch.Tensor, l: Layer) -> torch.Tensor:
    # window origin = -pad/2, out-of-image taps ignored (src-lib/maxpool_layer_kernels.cu:48-86)
    lo = l.pad // 2
    need_h = (l.out_h - 1) * l.stride + l.size - lo
    need_w = (l.out_w - 1) * l.stride + l.size - lo
    hi_w, hi_h = max(need_w - l.w, 0), max(need_h - l.h, 0)
    if lo or hi_w or hi_h:                                       # the common 2x2/stride-2 pool of an even map needs none
        x = F.pad(x, (lo, hi_w, lo, hi_h), value=float("-inf"))
    y = F.max_pool2d(x, l.size, l.stride)
    if y.shape[2] != l.out_h or y.shape[3] != l.out_w:
        y = y[:, :, :l.out_h, :l.out_w].contiguous()
    return y


def _yolo(x: torch.Tensor, l: Layer) -> torch.Tensor:
    # logistic on x, y, objectness and classes; w, h raw (src-lib/yolo_layer.cpp:1439-1489)
    mask = [int(v) for v in l.opts["mask"].split(",")]
    classes = int(l.opts.get("classes", 20))
    b = x.shape[0]
    if x.is_cuda and x.is_contiguous() and float(l.opts.get("scale_x_y", 1)) == 1.0:
        out = torch.empty_like(x)
        capi.check(capi.lib().xnor_b200_yolo_activate(x.data_ptr(), out.data_ptr(), b, len(mask), classes, l.h * l.w,
                                                     torch.cuda.current_stream().cuda_stream), "xnor_b200_yolo_activate")
        return out
    v = x.reshape(b, len(mask), 5 + classes, l.h * l.w).clone()
    v[:, :, 0:2] = torch.sigmoid(v[:, :, 0:2])
    v[:, :, 4:] = torch.sigmoid(v[:, :, 4:])
    return v.reshape(b, -1, l.h, l.w)


def _region(x: torch.Tensor, l: Layer) -> torch.Tensor:
    # logistic on x, y and objectness, softmax over classes (src-lib/region_layer.cpp:494-537)
    num = int(l.opts.get("num", 1))
    classes = int(l.opts.get("classes", 20))
    coords = int(l.opts.get("coords", 4))
    b = x.shape[0]
    if x.is_cuda and x.is_contiguous() and coords >= 2:
        out = torch.empty_like(x)
        capi.check(capi.lib().xnor_b200_region_activate(x.data_ptr(), out.data_ptr(), b, num, coords, classes, int(l.opts.get("softmax", 0)),
                                                       l.h * l.w, torch.cuda.current_stream().cuda_stream), "xnor_b200_region_activate")
        return out
    v = x.reshape(b, num, coords + 1 + classes, l.h * l.w).clone()
    v[:, :, 0:2] = torch.sigmoid(v[:, :, 0:2])
    v[:, :, coords] = torch.sigmoid(v[:, :, coords])
    if int(l.opts.get("softmax", 0)):
        v[:, :, coords + 1:] = torch.softmax(v[:, :, coords + 1:], dim=2)
    return v.reshape(b, -1, l.h, l.w)


def forward_network_gpu(net: Network, x: torch.Tensor, heads_host: Optional[List[torch.Tensor]] = None) -> List[torch.Tensor]:
    """The layer loop of forward_network_gpu (src-lib/network_kernels.cu:30-65).  Returns the outputs of the
    network's head layers (yolo / region / softmax).  heads_host: pinned host tensors, one per head; each head is
    copied there as soon as it exists, on the stream that made it (Darknet's yolo layer pulls its output to the host
    in every forward, src-lib/yolo_layer.cpp:1439-1489), so the copy of an early head overlaps the rest of the network."""
    heads: List[torch.Tensor] = []
    cur = x
    side_ctx = None
    joins: List[torch.cuda.Event] = []
    for l in net.layers:
        if l.branch_start and x.is_cuda:
            # fork: the side stream picks up after the layer that feeds both branches
            if net.side_stream is None:
                net.side_stream = torch.cuda.Stream(x.device)
            fork = torch.cuda.Event()
            fork.record(torch.cuda.current_stream())
            net.side_stream.wait_event(fork)
            side_ctx = torch.cuda.stream(net.side_stream)
            side_ctx.__enter__()
        if l.type == "convolutional":
            if l.xnor:
                xl = l.xnor_layer
                nxt = net.layers[l.index + 1] if l.index + 1 < len(net.layers) else None
                if nxt is not None and nxt.blank:
                    xl.bin_conv_shortcut_in_gpu = net.layers[nxt.input_layers[0]].output_gpu
                if l.emit_signs or l.sign_source is not None or l.mask_source is not None or l.sinks or l.packed_input or xl.window_major:
                    src = net.layers[l.sign_source].sign_out if l.sign_source is not None else None
                    masks = net.layers[l.mask_source].sign_out if l.mask_source is not None else None
                    want_fp32 = not l.emit_signs and (l.need_fp32 or not l.sinks)
                    so = l.shortcut_only and want_fp32 and not l.sinks
                    out = L.forward_convolutional_layer_io(xl, x=None if (src is not None or masks is not None or l.packed_input) else cur,
                                                           x_signs=src, pool=l.pool_desc, want_signs=l.emit_signs, packed=l.packed_input,
                                                           sinks=l.sinks, want_output=want_fp32, x_masks=masks, shortcut_only=so,
                                                           shortcut_signs=l.emit_sum_signs,
                                                           shortcut_sink=net.layers[l.sum_sink_to].xnor_layer if l.sum_sink_to is not None else None)
                    l.sign_out = out if l.emit_signs else None
                    cur = out if (want_fp32 and not so) else None
                elif l.shortcut_only or l.emit_sum_signs or l.sum_sink_to is not None:
                    out = L.forward_convolutional_layer_io(xl, x=cur, pool=l.pool_desc, shortcut_only=l.shortcut_only, want_output=True,
                                                           shortcut_signs=l.emit_sum_signs,
                                                           shortcut_sink=net.layers[l.sum_sink_to].xnor_layer if l.sum_sink_to is not None else None)
                    cur = None if l.shortcut_only else out
                else:
                    cur = L.forward_convolutional_layer_gpu(xl, cur, l.pool_desc)
            elif l.c == 3 and l.size == 3 and l.stride == 1 and l.pad == 1 and l.activation in ("leaky", "linear"):
                cur = _float_conv3(net, l, cur.contiguous())
                if l.emit_planes or l.emit_masks:
                    l.sign_out, cur = cur, None
            elif l.c * l.size * l.size <= 128 and l.n <= 256 and l.activation in ("leaky", "linear"):
                cur = _float_conv_small(net, l, cur)
            elif l.weights_blocked_gpu is not None:
                # a head whose yolo activation runs in this kernel can be written straight into the caller's pinned host tensor
                direct = heads_host is not None and l.yolo_entries > 0 and net.heads_direct_to_host
                cur = _float_conv_map(net, l, cur.contiguous(), heads_host[len(heads)] if direct else None)
            elif l.size == 1 and l.stride == 1 and l.pad == 0 and l.activation in ("leaky", "linear"):
                # a 1x1 convolution over many pixels: one GEMM over the whole batch on the tensor cores (three tf32 products
                # per operand pair), bias and activation in its epilogue
                cur = _float_conv_1x1_tc(l, cur.contiguous())
            elif l.size == 1 and l.stride == 1 and l.pad == 0:
                # other activations: a plain matrix product per image (cuBLAS sgemm, fp32)
                b = cur.shape[0]
                y = torch.baddbmm(l.biases_gpu.view(1, l.n, 1), l.weights_gpu.view(1, l.n, l.c).expand(b, -1, -1),
                                  cur.reshape(b, l.c, l.h * l.w))
                cur = _activate(y.view(b, l.n, l.out_h, l.out_w), l.activation)
            else:
                cur = _activate(F.conv2d(cur, l.weights_gpu, l.biases_gpu, l.stride, l.pad), l.activation)
        elif l.skip:
            cur = None                            # only sat between a sink producer and its consumer
        elif l.type == "maxpool":
            if not l.folded:                      # a folded maxpool hands its input on untouched
                cur = _maxpool(cur, l)
        elif l.type == "route":
            cur = net.layers[l.input_layers[0]].output_gpu if len(l.input_layers) == 1 else \
                torch.cat([net.layers[i].output_gpu for i in l.input_layers], 1)
        elif l.type == "shortcut":
            cur = l.output_gpu if l.blank else _activate(cur + net.layers[l.input_layers[0]].output_gpu, l.activation)
            prev = net.layers[l.index - 1]
            if l.blank and prev.emit_sum_signs:
                l.sign_out = prev.xnor_layer.shortcut_signs_gpu
        elif l.type == "upsample":
            cur = F.interpolate(cur, scale_factor=l.stride, mode="nearest")
        elif l.type == "avgpool":
            cur = cur.mean((2, 3), keepdim=True)
        elif l.type == "softmax":
            cur = torch.softmax(cur.reshape(cur.shape[0], -1), 1).reshape(cur.shape)
            heads.append(cur)
            if heads_host is not None:
                heads_host[len(heads) - 1].copy_(cur, non_blocking=True)
        elif l.type == "yolo":
            cur = cur if l.yolo_done else _yolo(cur, l)
            heads.append(cur)
            if heads_host is not None and cur is not heads_host[len(heads) - 1]:
                heads_host[len(heads) - 1].copy_(cur, non_blocking=True)
        elif l.type == "region":
            cur = _region(cur, l)
            heads.append(cur)
            if heads_host is not None:
                heads_host[len(heads) - 1].copy_(cur, non_blocking=True)
        l.output_gpu = cur
        if l.branch_end and side_ctx is not None:
            done = torch.cuda.Event()
            done.record(net.side_stream)
            joins.append(done)
            side_ctx.__exit__(None, None, None)
            side_ctx = None
    for done in joins:                                # join: the caller's stream sees both branches finished
        torch.cuda.current_stream().wait_event(done)
    return heads


# ---- detections ----------------------------------------------------------------------------------

class DetectionBuffers:
    """Device buffers of xnor_b200_detections plus the row list: one detection list per image of the batch."""

    def __init__(self, batch: int, classes: int, max_dets: int = 2048, max_rows: int = 4096, device="cuda:0") -> None:
        self.batch, self.classes, self.max_dets, self.max_rows = batch, classes, max_dets, max_rows
        self.boxes = torch.empty(batch, max_dets, 4, dtype=torch.float32, device=device)
        self.objectness = torch.empty(batch, max_dets, dtype=torch.float32, device=device)
        self.probs = torch.empty(batch, max_dets, classes, dtype=torch.float32, device=device)
        self.count = torch.zeros(batch, dtype=torch.int32, device=device)
        self.rows = torch.empty(batch, max_rows, 7, dtype=torch.float32, device=device)
        self.row_count = torch.zeros(batch, dtype=torch.int32, device=device)
        self.desc = capi.Detections(self.boxes.data_ptr(), self.objectness.data_ptr(), self.probs.data_ptr(), self.count.data_ptr(),
                                    max_dets, classes)

    def rows_host(self) -> List[np.ndarray]:
        """Per image the rows {x, y, w, h, objectness, class, probability} (one device-to-host copy of the counts, one of the rows)."""
        counts = self.row_count.cpu().numpy()
        rows = self.rows.cpu().numpy()
        return [rows[b, :min(int(counts[b]), self.max_rows)].copy() for b in range(self.batch)]


def yolo_head_desc(l: Layer, output: torch.Tensor) -> capi.YoloHead:
    """The [yolo] section's own anchors (biases[2 * mask[a]], src-lib/yolo_layer.cpp:22-42) and sizes for xnor_b200_yolo_detections."""
    mask = [int(v) for v in l.opts["mask"].split(",")]
    anchors = [float(v) for v in l.opts["anchors"].split(",")]
    hd = capi.YoloHead()
    hd.output = output.data_ptr()
    hd.w, hd.h, hd.n, hd.classes = l.w, l.h, len(mask), int(l.opts.get("classes", 20))
    for a, m in enumerate(mask):
        hd.anchors[2 * a], hd.anchors[2 * a + 1] = anchors[2 * m], anchors[2 * m + 1]
    hd.new_coords = int(l.opts.get("new_coords", 0))
    return hd


def get_network_boxes(net: Network, heads: List[torch.Tensor], img_w: int, img_h: int, thresh: float, dets: DetectionBuffers,
                      relative: int = 1, letter: int = 0) -> DetectionBuffers:
    """get_network_boxes (src-lib/darknet_network.cpp:1250) on the device: every [yolo] head of the network, in layer order, appended
    to one detection list per image.  `heads` are the activated head outputs forward_network_gpu returned (device tensors)."""
    import ctypes as C
    yolo_layers = [l for l in net.layers if l.type == "yolo"]
    if len(yolo_layers) != len(heads) or not yolo_layers:
        raise ValueError("one activated output per [yolo] layer is needed")
    stream = torch.cuda.current_stream().cuda_stream
    for k, (l, h) in enumerate(zip(yolo_layers, heads)):
        if not (h.is_cuda and h.is_contiguous() and h.dtype == torch.float32):
            raise ValueError("head outputs must be contiguous fp32 device tensors")
        hd = yolo_head_desc(l, h)
        capi.check(capi.lib().xnor_b200_yolo_detections(C.byref(hd), net.batch, net.w, net.h, img_w, img_h, thresh, relative, letter,
                                                       1 if k else 0, C.byref(dets.desc), stream), "xnor_b200_yolo_detections")
    return dets


def do_nms_sort(dets: DetectionBuffers, nms_thresh: float) -> None:
    """do_nms_sort (src-lib/box.cpp:951) on the device, every image and class at once."""
    import ctypes as C
    capi.check(capi.lib().xnor_b200_nms_sort(C.byref(dets.desc), dets.batch, nms_thresh, torch.cuda.current_stream().cuda_stream),
               "xnor_b200_nms_sort")


def detection_rows(dets: DetectionBuffers) -> None:
    """Fills dets.rows / dets.row_count with the surviving (detection, class) pairs."""
    import ctypes as C
    capi.check(capi.lib().xnor_b200_detection_rows(C.byref(dets.desc), dets.batch, dets.rows.data_ptr(), dets.max_rows,
                                                  dets.row_count.data_ptr(), torch.cuda.current_stream().cuda_stream), "xnor_b200_detection_rows")


def network_detections(net: Network, x: torch.Tensor, thresh: float = 0.25, nms_thresh: float = 0.45,
                       dets: Optional[DetectionBuffers] = None, img_w: Optional[int] = None, img_h: Optional[int] = None) -> DetectionBuffers:
    """Forward + decode + suppress + compact, all on the device: what a caller of Darknet's predict API does with
    network_predict, get_network_boxes and do_nms_sort.  The result's rows are the only thing that has to cross to the host."""
    heads = forward_network_gpu(net, x)
    if dets is None:
        classes = int(next(l for l in net.layers if l.type == "yolo").opts.get("classes", 20))
        dets = DetectionBuffers(net.batch, classes, device=x.device)
    get_network_boxes(net, heads, img_w or net.w, img_h or net.h, thresh, dets)
    if nms_thresh > 0:
        do_nms_sort(dets, nms_thresh)
    detection_rows(dets)
    return dets


def load_network_custom(cfg: str, weights: str, batch: int = 1, device: str = "cuda:0", sign_chains: bool = True,
                        fuse_first_conv: bool = True, side_branches: bool = True, float_map_max_pixels: Optional[int] = None,
                        sum_signs_min_batch: Optional[int] = None, sink_max_batch: Optional[int] = None,
                        packed_cache: bool = False) -> Network:
    """load_network_custom (src-lib/weights.cpp:665-691): parse, load, fold batch-norm, pack binary weights.
    float_map_max_pixels, sum_signs_min_batch and sink_max_batch override the measured hand-over thresholds of the Network
    (tuning runs).  packed_cache: read the packed weights from <weights>.xnorpack where it matches, and (re)write that file
    when any layer had to be packed afresh."""
    torch.backends.cudnn.allow_tf32 = False
    torch.backends.cuda.matmul.allow_tf32 = False
    net = parse_network_cfg(cfg, batch, device)
    net.sign_chains = sign_chains
    net.skip_fused_conv_outputs = sign_chains      # the plain network keeps every layer's own tensor
    net.fuse_first_conv = fuse_first_conv
    net.side_branches = side_branches
    if float_map_max_pixels is not None:
        net.float_map_max_pixels = float_map_max_pixels
    if sum_signs_min_batch is not None:
        net.sum_signs_min_batch = sum_signs_min_batch
    if sink_max_batch is not None:
        net.sink_max_batch = sink_max_batch
    load_weights(net, weights)
    fuse_conv_batchnorm(net)
    packed = None
    if packed_cache and os.path.exists(packed_cache_path(weights)):
        try:
            packed = read_packed_cache(packed_cache_path(weights))
        except (OSError, ValueError):
            packed = None                    # unusable file: pack afresh and replace it
    calculate_binary_weights(net, packed)
    n_xnor = sum(1 for l in net.layers if l.type == "convolutional" and l.xnor)
    if packed_cache and net.packed_from_cache < n_xnor:
        write_packed_cache(packed_cache_path(weights), packed_entries(net))
    return net


def own_launches_per_forward(net: Network) -> int:
    """Kernels of libxnor_b200.so that one forward launches, after every fusion that load_network_custom set up."""
    n = 0
    for l in net.layers:
        if l.type == "convolutional":
            if l.xnor:
                # GEMM (+ pack kernel); the short-K GEMM builds its rows from the first conv's sign planes itself
                from_planes = l.mask_source is not None or (
                    l.sign_source is not None and l.c % 32 != 0 and (l.size, l.stride, l.pad) == (3, 1, 1) and l.c * 9 <= 256)
                n += 1 if (l.packed_input or from_planes) else 2
            elif (l.c == 3 and l.size == 3 and l.stride == 1 and l.pad == 1) or l.c * l.size * l.size <= 128 or l.weights_blocked_gpu is not None:
                n += 1
            elif l.size == 1 and l.stride == 1 and l.pad == 0 and l.activation in ("leaky", "linear"):
                n += 1                                    # tensor-core 1x1 float convolution
        elif (l.type == "yolo" and not l.yolo_done) or l.type == "region":
            n += 1
    return n


def xnor_layer_shapes(net: Network) -> List[dict]:
    """Per xnor layer: GEMM sizes and binary-op count per image (2*M*N*K, unpadded K)."""
    rows = []
    for l in net.layers:
        if l.type == "convolutional" and l.xnor:
            M, N, K = l.n, l.out_h * l.out_w, l.size * l.size * l.c
            rows.append(dict(index=l.index, c=l.c, h=l.h, w=l.w, n=l.n, size=l.size, stride=l.stride, pad=l.pad,
                             activation=l.activation, M=M, N=N, K=K, binops=2 * M * N * K))
    return rows
