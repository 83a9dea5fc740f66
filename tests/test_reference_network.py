"""The reference's OWN network code (cfg parser, .weights loader, fuse_conv_batchnorm, calculate_binary_weights, every layer's
CPU forward: oracle/_ref/liboracle_refnet.so, built by oracle/build_refnet.py from the mounted darknet tree) against the
host-side mirror in darknet_b200/network.py and against the oracle restatement -- on the CPU, no GPU involved.  Skipped where
that library has not been built."""
import numpy as np
import pytest

import synth

torch = pytest.importorskip("torch")

from darknet_b200 import cfgs, network  # noqa: E402
from oracle.binding import RefNet  # noqa: E402

pytestmark = pytest.mark.skipif(not RefNet.available(), reason="oracle/_ref/liboracle_refnet.so not built (python oracle/build_refnet.py)")

LINEAR, LEAKY = 4, 9          # the reference's ACTIVATION enum (include/darknet.h)


def make(tmp_path, name, size, seed, **kw):
    cfg, w = tmp_path / "net.cfg", tmp_path / "net.weights"
    cfg.write_text(cfgs.CFGS[name](size, size))
    net = network.parse_network_cfg(str(cfg), 1, "cpu")
    network.write_synthetic_weights(net, str(w), seed=seed, **kw)
    network.load_weights(net, str(w))
    return str(cfg), str(w), net


@pytest.mark.parametrize("name", ["yolov3-tiny_xnor", "tiny-yolo_xnor", "darknet53_448_xnor"])
def test_batchnorm_fold_and_activation_rule_equal_the_reference(tmp_path, name):
    """fuse_conv_batchnorm (src-lib/darknet_network.cpp:1667-1708) with random batch-norm statistics: folded weights and
    biases bit for bit; calculate_binary_weights' rule (:1794-1797): a bin_output xnor layer ends up LINEAR."""
    cfg, w, net = make(tmp_path, name, 64, 5, random_batchnorm=True)
    ref = RefNet(cfg, w, 1)
    network.fuse_conv_batchnorm(net)
    assert ref.n == len(net.layers)
    checked = 0
    for i, l in enumerate(net.layers):
        info = ref.layer_info(i)
        if l.type != "convolutional":
            continue
        rw, rb = ref.layer_weights(i, l.weights.size, l.n)
        assert np.array_equal(rw.view(np.uint32), l.weights.reshape(-1).view(np.uint32)), f"folded weights of layer {i} differ"
        assert np.array_equal(rb.view(np.uint32), l.biases.view(np.uint32)), f"folded biases of layer {i} differ"
        assert info["xnor"] == l.xnor and info["packed"] == l.xnor
        if l.xnor:
            want = "linear" if l.use_bin_output else l.activation
            assert info["activation"] == {"linear": LINEAR, "leaky": LEAKY}[want], f"activation of xnor layer {i}"
        checked += 1
    assert checked > 5
    ref.close()


@pytest.mark.parametrize("name,size", [("yolov3-tiny_xnor", 96), ("tiny-yolo_xnor", 96), ("darknet53_448_xnor", 64)])
def test_restatement_equals_the_reference_inside_a_network(tmp_path, port, name, size):
    """Every xnor layer of a whole reference forward: the oracle restatement, fed the tensor the reference layer saw and the
    folded weights, reproduces the reference layer's output bit for bit (fused [shortcut] sums aside, which the CPU
    reference does not fuse)."""
    cfg, w, net = make(tmp_path, name, size, 7, random_batchnorm=True)
    ref = RefNet(cfg, w, 1)
    network.fuse_conv_batchnorm(net)
    x = synth.uniform01(31, (1, 3, size, size))
    ref.predict(x)
    checked = 0
    for i, l in enumerate(net.layers):
        if not (l.type == "convolutional" and l.xnor):
            continue
        src = ref.layer_output(i - 1)
        leaky = (l.activation == "leaky") and not l.use_bin_output
        want = ref.layer_output(i)
        got = port.conv_forward(np.ascontiguousarray(src), l.weights, l.biases, l.stride, l.pad, leaky)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), f"xnor layer {i}: restatement differs from the reference"
        checked += 1
    assert checked == sum(1 for l in net.layers if l.type == "convolutional" and l.xnor)
    ref.close()
