"""The three xnor networks end to end against the REFERENCE's own network code on the CPU (load_network_custom ->
network_predict of oracle/_ref/liboracle_refnet.so, built by oracle/build_refnet.py): the same .cfg text and the same
.weights file go to both sides.

The float convolution in front of the first xnor layer adds its 27 products in a different order on the two sides, and an
activation within rounding of zero would then binarise differently.  Instead of tolerating that, the weights file makes the
first convolution exact (weights and biases on a 2^-10 grid, inputs on a 2^-8 grid: every partial sum is representable), so
both sides binarise bit-identical tensors; every xnor layer must then equal the reference's layer output bit for bit, all the
way down the network, and the head outputs must agree within 1e-3 -- every value."""
import numpy as np
import pytest

import synth

torch = pytest.importorskip("torch")
pytestmark = [pytest.mark.gpu]

from darknet_b200 import cfgs, network  # noqa: E402
from oracle.binding import RefNet  # noqa: E402

if not RefNet.available():
    pytest.skip("oracle/_ref/liboracle_refnet.so not built (python oracle/build_refnet.py, needs the reference tree)", allow_module_level=True)


@pytest.mark.parametrize("name,size", [("yolov3-tiny_xnor", 416), ("tiny-yolo_xnor", 416), ("darknet53_448_xnor", 448), ("darknet53_448_xnor", 128)])
def test_network_equals_the_reference_network(tmp_path, name, size):
    cfg, w = tmp_path / "net.cfg", tmp_path / "net.weights"
    cfg.write_text(cfgs.CFGS[name](size, size))
    net_cpu = network.parse_network_cfg(str(cfg), 1, "cpu")
    network.write_synthetic_weights(net_cpu, str(w), seed=19, random_batchnorm=True, exact_first_conv=True)
    x = np.floor(synth.uniform01(29, (1, 3, size, size)) * 256.0).astype(np.float32) / 256.0
    ref = RefNet(str(cfg), str(w), 1)
    ref.predict(x)

    plain = network.load_network_custom(str(cfg), str(w), 1, sign_chains=False, fuse_first_conv=False, side_branches=False)
    heads = [h.cpu().numpy() for h in network.forward_network_gpu(plain, torch.from_numpy(x).cuda())]
    first = next(i for i, l in enumerate(plain.layers) if l.type == "convolutional" and l.xnor)
    got_in = plain.layers[first - 1].output_gpu.cpu().numpy()
    want_in = ref.layer_output(first - 1)
    assert np.array_equal(got_in.view(np.uint32), want_in.view(np.uint32)), "the exact first convolution is not exact"
    checked = 0
    for i, l in enumerate(plain.layers):
        if l.type == "convolutional" and l.xnor:
            got = l.xnor_layer.output_gpu.cpu().numpy()
            want = ref.layer_output(i)
            assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), f"xnor layer {i} differs from the reference network"
            checked += 1
        elif l.type == "shortcut":
            got, want = l.output_gpu.cpu().numpy(), ref.layer_output(i)
            assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), f"[shortcut] {i} differs from the reference network"
    assert checked == sum(1 for l in plain.layers if l.type == "convolutional" and l.xnor)

    head_layers = [i for i, l in enumerate(plain.layers) if l.type in ("yolo", "region", "softmax")]
    assert len(head_layers) == len(heads) > 0
    for i, h in zip(head_layers, heads):
        want = ref.layer_output(i).reshape(h.shape)
        if plain.layers[i].type == "region":
            # The reference's CPU region layer leaves its output cell-major ([cell][anchor][entry], flatten() in
            # src-lib/region_layer.cpp:216) and applies the logistic of x and y only later, inside get_region_box (:92-93);
            # the device kernel keeps Darknet's [anchor][entry][cell] layout and applies it at once.  Same numbers, re-ordered.
            o = plain.layers[i].opts
            num, size_ = int(o.get("num", 1)), int(o.get("coords", 4)) + 1 + int(o.get("classes", 20))
            r = ref.layer_output(i).reshape(-1, num, size_).transpose(1, 2, 0).copy()
            r[:, 0:2] = 1.0 / (1.0 + np.exp(-r[:, 0:2].astype(np.float64)))
            want = r.astype(np.float32).reshape(h.shape)
        worst = float(np.abs(h - want).max())
        assert worst <= 1e-3, f"head {i} differs from the reference by {worst:.3e}"

    # the linked network (every fusion on) reaches the same heads bit for bit
    linked = network.load_network_custom(str(cfg), str(w), 1)
    for a, b in zip(network.forward_network_gpu(linked, torch.from_numpy(x).cuda()), heads):
        assert np.array_equal(a.cpu().numpy().view(np.uint32), b.view(np.uint32))
    ref.close()


def test_device_detections_equal_the_reference_end_to_end(tmp_path):
    """network_detections (forward, decode, suppress, compact: all on the device) against network_predict +
    get_network_boxes + do_nms_sort of the reference on the same file: same (class, cell) set; probabilities within 1e-3."""
    size = 416
    cfg, w = tmp_path / "net.cfg", tmp_path / "net.weights"
    cfg.write_text(cfgs.yolov3_tiny_xnor_cfg(size, size))
    net_cpu = network.parse_network_cfg(str(cfg), 1, "cpu")
    network.write_synthetic_weights(net_cpu, str(w), seed=23, exact_first_conv=True)
    x = np.floor(synth.uniform01(3, (1, 3, size, size)) * 256.0).astype(np.float32) / 256.0
    ref = RefNet(str(cfg), str(w), 1)
    ref.predict(x)
    thresh = 0.9
    want = ref.detections(size, size, thresh, 0.0)
    ref.close()
    net = network.load_network_custom(str(cfg), str(w), 1)
    dets = network.network_detections(net, torch.from_numpy(x).cuda(), thresh=thresh, nms_thresh=0.0)
    torch.cuda.synchronize()
    got = dets.rows_host()[0]
    assert len(want) > 20
    # The float head convolutions round differently on the two sides (1e-6 .. 1e-4), which can carry a value across the
    # threshold; so rows are matched (same class, box within 1e-3) and a row without a partner must sit on the threshold.
    used = np.zeros(len(got), bool)
    unmatched = []
    for r in want:
        cand = np.where((got[:, 5] == r[5]) & ~used & (np.abs(got[:, :4] - r[:4]).max(1) <= 1e-3))[0]
        if len(cand):
            used[cand[0]] = True
            assert np.abs(got[cand[0]] - r).max() <= 1e-3
        else:
            unmatched.append(r)
    unmatched += list(got[~used])
    assert len(unmatched) <= max(2, len(want) // 50), f"{len(unmatched)} of {len(want)} rows have no partner"
    for r in unmatched:
        assert min(abs(r[6] - thresh), abs(r[4] - thresh)) <= 2e-3, "an unmatched row that is not a threshold case"
