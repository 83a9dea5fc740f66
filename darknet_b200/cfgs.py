"""Generators for the three xnor network descriptions Darknet ships, in Darknet's own .cfg syntax.

The benchmark box has no copy of the reference tree, so the cfg text is produced here from the
published topologies and then parsed by the same parser that reads a real .cfg file.  A CPU test
checks, where the reference tree is mounted, that each generated text parses to exactly the layer list
of the corresponding cfg/*.cfg file (section types, sizes, xnor and bin_output flags, activations,
route/shortcut sources, head parameters).
"""
from __future__ import annotations

from typing import List

_YOLO_ANCHORS = "10,14,  23,27,  37,58,  81,82,  135,169,  344,319"
_REGION_ANCHORS = "0.738768,0.874946,  2.42204,2.65704,  4.30971,7.04493,  10.246,4.59428,  12.6868,11.8741"


def _conv(filters: int, size: int, stride: int = 1, xnor: int = 0, bin_output: int = 0, bn: int = 1, activation: str = "leaky") -> str:
    lines = ["[convolutional]"]
    if xnor:
        lines.append("xnor=1")
    if bin_output:
        lines.append("bin_output=1")
    if bn:
        lines.append("batch_normalize=1")
    lines += [f"filters={filters}", f"size={size}", f"stride={stride}", "pad=1", f"activation={activation}", ""]
    return "\n".join(lines)


def _maxpool(size: int, stride: int) -> str:
    return f"[maxpool]\nsize={size}\nstride={stride}\n"


def yolov3_tiny_xnor_cfg(width: int = 416, height: int = 416) -> str:
    """yolov3-tiny with xnor=1 on the inner convolutions; two yolo heads (13x13 and 26x26 at 416)."""
    s: List[str] = [f"[net]\nbatch=1\nsubdivisions=1\nwidth={width}\nheight={height}\nchannels=3\n"]
    s += [_conv(16, 3), _maxpool(2, 2)]
    s += [_conv(32, 3, xnor=1, bin_output=1), _maxpool(2, 2)]
    s += [_conv(64, 3, xnor=1, bin_output=1), _maxpool(2, 2)]
    s += [_conv(128, 3, xnor=1, bin_output=1), _maxpool(2, 2)]
    s += [_conv(256, 3, xnor=1), _maxpool(2, 2)]
    s += [_conv(512, 3, xnor=1, bin_output=1), _maxpool(2, 1)]
    s += [_conv(1024, 3, xnor=1, bin_output=1)]
    s += [_conv(256, 1, xnor=1)]
    s += [_conv(512, 3)]
    s += [_conv(255, 1, bn=0, activation="linear")]
    s += [f"[yolo]\nmask = 3,4,5\nanchors = {_YOLO_ANCHORS}\nclasses=80\nnum=6\n"]
    s += ["[route]\nlayers = -4\n"]
    s += [_conv(128, 1, xnor=1)]
    s += ["[upsample]\nstride=2\n"]
    s += ["[route]\nlayers = -1, 8\n"]
    s += [_conv(256, 3, xnor=1)]
    s += [_conv(255, 1, bn=0, activation="linear")]
    s += [f"[yolo]\nmask = 0,1,2\nanchors = {_YOLO_ANCHORS}\nclasses=80\nnum=6\n"]
    return "\n".join(s)


def tiny_yolo_xnor_cfg(width: int = 416, height: int = 416) -> str:
    """YOLOv2-tiny topology with xnor=1 on the inner convolutions and a region head (5 anchors, 80 classes)."""
    s: List[str] = [f"[net]\nbatch=1\nsubdivisions=1\nwidth={width}\nheight={height}\nchannels=3\n"]
    s += [_conv(16, 3), _maxpool(2, 2)]
    for f in (32, 64, 128, 256):
        s += [_conv(f, 3, xnor=1, bin_output=1), _maxpool(2, 2)]
    s += [_conv(512, 3, xnor=1, bin_output=1), _maxpool(2, 1)]
    s += [_conv(1024, 3, xnor=1, bin_output=1)]
    s += [_conv(1024, 3, xnor=1)]
    s += [_conv(425, 1, bn=0, activation="linear")]
    s += [f"[region]\nanchors = {_REGION_ANCHORS}\nbias_match=1\nclasses=80\ncoords=4\nnum=5\nsoftmax=1\n"]
    return "\n".join(s)


def darknet53_448_xnor_cfg(width: int = 448, height: int = 448) -> str:
    """Darknet-53 classifier with xnor=1 on every convolution of the residual trunk."""
    s: List[str] = [f"[net]\nbatch=1\nsubdivisions=1\nheight={height}\nwidth={width}\nchannels=3\n"]
    s += [_conv(32, 3)]
    for filters, blocks in ((64, 1), (128, 2), (256, 8), (512, 8), (1024, 4)):
        s += [_conv(filters, 3, stride=2, xnor=1)]
        for _ in range(blocks):
            s += [_conv(filters // 2, 1, xnor=1), _conv(filters, 3, xnor=1), "[shortcut]\nfrom=-3\nactivation=linear\n"]
    s += [_conv(512, 1)]
    s += ["[avgpool]\n"]
    s += [_conv(1000, 1, bn=0, activation="linear")]
    s += ["[softmax]\ngroups=1\n"]
    return "\n".join(s)


CFGS = {
    "yolov3-tiny_xnor": yolov3_tiny_xnor_cfg,
    "tiny-yolo_xnor": tiny_yolo_xnor_cfg,
    "darknet53_448_xnor": darknet53_448_xnor_cfg,
}
