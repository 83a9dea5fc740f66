"""CPU checks of the host logic around the path: cfg parsing, the generated cfg texts against the
reference's shipped cfg files, .weights round trip, batch-norm folding and the bin_output rules."""
import os

import numpy as np
import pytest

torch = pytest.importorskip("torch")
from darknet_b200 import cfgs, network  # noqa: E402

from oracle.binding import reference_dir  # noqa: E402

REF_CFG = os.path.join(reference_dir(), "cfg")


def parse_text(text, tmp_path, name="net.cfg"):
    p = tmp_path / name
    p.write_text(text)
    return network.parse_network_cfg(str(p), 1, "cpu")


def summary(net):
    rows = []
    for l in net.layers:
        rows.append((l.type, l.c, l.h, l.w, l.out_c, l.out_h, l.out_w, l.n, l.size, l.stride, l.pad, l.activation if l.type in ("convolutional", "shortcut") else "",
                     l.batch_normalize, l.xnor, l.use_bin_output, tuple(l.input_layers),
                     tuple(sorted((k, v.replace(" ", "")) for k, v in l.opts.items() if k in ("mask", "anchors", "classes", "num", "coords", "softmax")))))
    return rows


@pytest.mark.parametrize("name", list(cfgs.CFGS))
def test_generated_cfg_equals_shipped_cfg(name, tmp_path):
    ref_file = os.path.join(REF_CFG, name + ".cfg")
    if not os.path.exists(ref_file):
        pytest.skip("reference tree not mounted")
    ours = parse_text(cfgs.CFGS[name](), tmp_path)
    theirs = network.parse_network_cfg(ref_file, 1, "cpu")
    assert (ours.c, ours.h, ours.w) == (theirs.c, theirs.h, theirs.w)
    assert summary(ours) == summary(theirs)


def test_xnor_layer_tables_match_the_published_shapes(tmp_path):
    net = parse_text(cfgs.yolov3_tiny_xnor_cfg(), tmp_path)
    for l in net.layers:
        l.xnor and setattr(l, "weights", None)
    rows = network.xnor_layer_shapes(net)
    assert [(r["index"], r["c"], r["M"], r["N"], r["K"]) for r in rows] == [
        (2, 16, 32, 43264, 144), (4, 32, 64, 10816, 288), (6, 64, 128, 2704, 576), (8, 128, 256, 676, 1152), (10, 256, 512, 169, 2304),
        (12, 512, 1024, 169, 4608), (13, 1024, 256, 169, 1024), (18, 256, 128, 169, 256), (21, 384, 256, 676, 3456)]
    assert sum(r["binops"] for r in rows) == 4884332544
    net = parse_text(cfgs.tiny_yolo_xnor_cfg(), tmp_path, "b.cfg")
    assert sum(r["binops"] for r in network.xnor_layer_shapes(net)) == 6778257408
    net = parse_text(cfgs.darknet53_448_xnor_cfg(), tmp_path, "c.cfg")
    rows = network.xnor_layer_shapes(net)
    assert len(rows) == 51
    assert abs(sum(r["binops"] for r in rows) / 1e9 - 56.518) < 0.01


def test_bin_output_is_cleared_by_route_and_shortcut(tmp_path):
    net = parse_text(cfgs.yolov3_tiny_xnor_cfg(), tmp_path)
    # layer 8 (conv256) has no bin_output in the cfg; layers 2,4,6,10,12 keep theirs; nothing routed has it
    assert [l.use_bin_output for l in net.layers if l.type == "convolutional"] == [0, 1, 1, 1, 0, 1, 1, 0, 0, 0, 0, 0, 0]
    text = "[net]\nwidth=8\nheight=8\nchannels=32\n[convolutional]\nxnor=1\nbin_output=1\nfilters=32\nsize=3\nstride=1\npad=1\nactivation=leaky\n" \
           "[convolutional]\nxnor=1\nbin_output=1\nfilters=32\nsize=3\nstride=1\npad=1\nactivation=leaky\n[shortcut]\nfrom=-2\nactivation=linear\n"
    net = parse_text(text, tmp_path, "d.cfg")
    assert [l.use_bin_output for l in net.layers[:2]] == [0, 0]


def test_weights_file_round_trip_and_bn_fold(tmp_path):
    net = parse_text(cfgs.yolov3_tiny_xnor_cfg(64, 64), tmp_path)
    w = tmp_path / "t.weights"
    network.write_synthetic_weights(net, str(w), seed=3)
    network.load_weights(net, str(w))
    conv = [l for l in net.layers if l.type == "convolutional"]
    assert conv[0].weights.shape == (16, 3, 3, 3) and conv[0].scales is not None and conv[-1].scales is None
    expected = 20 + sum(4 * (l.n * (4 if l.batch_normalize else 1) + l.n * l.c * l.size * l.size) for l in conv)
    assert os.path.getsize(w) == expected
    l = conv[1]
    l.scales = np.linspace(0.5, 1.5, l.n).astype(np.float32)
    l.rolling_mean = np.linspace(-1, 1, l.n).astype(np.float32)
    l.rolling_variance = np.linspace(0.25, 4, l.n).astype(np.float32)
    w0, b0 = l.weights.copy(), l.biases.copy()
    network.fuse_conv_batchnorm(net)
    std = np.sqrt(l.rolling_variance.astype(np.float64) + 0.00001)
    assert np.array_equal(l.weights, (w0.astype(np.float64) * (l.scales / std)[:, None, None, None]).astype(np.float32))
    assert np.array_equal(l.biases, (b0.astype(np.float64) - l.scales.astype(np.float64) * l.rolling_mean / std).astype(np.float32))
    assert all(x.batch_normalize == 0 for x in conv)


def test_maxpool_follows_darknet_padding_rule():
    l = network.Layer("maxpool", 0, 1, 5, 5, size=2, stride=1, pad=1, out_c=1, out_h=5, out_w=5)
    x = torch.arange(25.0).reshape(1, 1, 5, 5)
    y = network._maxpool(x, l)
    assert y.shape == (1, 1, 5, 5)
    assert y[0, 0, 4, 4] == 24 and y[0, 0, 0, 0] == 6 and y[0, 0, 4, 0] == 21
    l = network.Layer("maxpool", 0, 1, 6, 6, size=2, stride=2, pad=1, out_c=1, out_h=3, out_w=3)
    y = network._maxpool(torch.arange(36.0).reshape(1, 1, 6, 6), l)
    assert y.flatten().tolist() == [7, 9, 11, 19, 21, 23, 31, 33, 35]
